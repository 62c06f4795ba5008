"""Benchmark of the hot path: the fused i-attention component on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the reference's headline attention case): one head, seq_q = seq_kv = 16384, head dim
128, fp32 Q/K/V ~ N(0,1) from seed 3 with Q scaled by 1/sqrt(128), no mask.  A step
is one invocation of the compiled README attention component on one head.  At
N > 1 every rank runs its own head per step (heads are the independent units,
weak scaling) and the outputs are all-gathered over NCCL on a side stream so the
gather of step s overlaps the kernel of step s+1.  Inputs rotate over several
distinct sets whose total size exceeds L2, so no step starts with its operands
cached.

One JSON line is printed by rank 0:
  value      TFLOP/s over all ranks with inputs resident in HBM (4*Nq*Nk*d FLOP
             per head), timed with CUDA events, max over ranks
  e2e        the same metric through the host-pointer C ABI (i_exec_into): every
             step copies Q, K, V from pinned host memory and O back
  roofline   tensor-bound: achieved = FLOP per step / average step time; the
             peak is MEASURED_PEAKS.json's dense bf16 figure for the default arm
             (fp16 operands issue at the bf16 rate) and for --precision bf16,
             half of it for --precision tf32 (the TF32 MMA issues at half that rate)
  sustained  the same loop run for about two seconds (the 200-step region lasts
             ~40 ms, too short for the power cap to bite)
  heads64_seq32768  the reference's multi-head case: 64 heads x 32768 x 128 divided
             over the ranks through i_b200.sharding, with and without the assembly
             of the output on every rank
  cpu_baseline  the reference's own emitted C (oracle/_ref) on the host cores,
             on a bounded row sample of the same workload
--impl reference times only that CPU program (rank 0; other ranks exit).
--only NAME runs one of the side measurements alone (a short run for a profiler).
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SEQ, DIM = 16384, 128
HEADS = 1             # heads per rank per step (one component invocation)
FLOP_PER_HEAD = 4.0 * SEQ * SEQ * DIM
METRIC = "fused i-attention TFLOP/s at seq16K d128"
WORKLOAD = "config4: single-head fused i-attention, seq_q=seq_kv=16384, d=128, fp32 N(0,1) seed 3, Q*1/sqrt(128)"
ROTATION = 8          # distinct input sets: 8 x 32 MiB = 256 MiB > 126 MB L2
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the attention kernel on this
# workload, from the ncu captures summarised in profiles/attention_pipelined_kernel_seq16384_d128.md
# (fp16 arm) and profiles/attention_tf32_kernel_seq16384_d128.md (the arms with 32-bit operands).
ATTENTION_DRAM_BYTES_PER_LAUNCH = {"f16": 17025024, "tf32+f16": 21210624, "tf32": 25411584}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


def make_inputs(seed=3, heads=1):
    import numpy as np
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((heads, SEQ, DIM), dtype=np.float32)
    k = rng.standard_normal((heads, SEQ, DIM), dtype=np.float32)
    v = rng.standard_normal((heads, SEQ, DIM), dtype=np.float32)
    q *= np.float32(1.0 / np.sqrt(DIM))
    return q, k, v


def readme_attention(ilang, batched=False):
    """The README attention component; with `batched`, the same chain with a
    leading head axis `h` so several heads are one invocation."""
    i, I = ilang.i, ilang.I
    h = "h" if batched else ""

    def e(src):
        # Prefix every index pattern and the loop order with the head axis.
        if not h:
            return i(src)
        expr, splits, order = (part.strip() for part in src.split("|"))
        out = ""
        for tok in expr.replace("~", " ~ ").replace("*", " * ").replace("-", " - ").replace(
                "/", " / ").split():
            out += (h + tok) if tok.isalpha() else tok
        for op in "+>^":
            if expr.startswith(op):
                out = op + h + out[len(op):]
        return i("%s | %s | %s" % (out, splits, h + order))

    mm_t = e("ik*jk~ijk | i:16,j:16 | jii'j'k") >> e("+ijk~ij | i:16,j:16 | jii'j'k0")
    row_max_shift = (I & e(">ij~i | i:16,j:16 | ji0i'j'")) >> e("ij-i~ij | i:16,j:16 | ji01i'j'")
    exp = e("^ij~ij | i:16,j:16 | ji0i'j'")
    row_normalize = (I & e("+ij~i | i:16,j:16 | ji0i'j'")) >> e("ij/i~ij | i:16,j:16 | ji01i'j'")
    mm = e("ij*jk~ikj | i:16,j:16 | ji0i'kj'") >> e("+ikj~ik | i:16,j:16 | jii'kj'0")
    return mm_t >> row_max_shift >> exp >> row_normalize >> mm


# ---------------------------------------------------------------------------
# CPU arm: the reference's own emitted C on the host cores.
# ---------------------------------------------------------------------------

def cpu_reference_sample(rows_per_core, repeats=1):
    """Times oracle/_ref (or the restated oracle when _ref is absent) on
    cores x rows_per_core query rows against all the keys of one head."""
    import numpy as np
    import oracle
    cores = os.cpu_count() or 1
    q, k, v = make_inputs()
    q, k, v = q[0], k[0], v[0]
    kind = "reference" if oracle.have_reference() else "port"
    fn = oracle.reference_attention if kind == "reference" else oracle.attention_fused
    stride = SEQ // cores
    blocks = [(c * stride, c * stride + rows_per_core) for c in range(cores)]
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.reference_attention_rows(q, k, v, blocks, threads=cores, fn=fn)
        times.append(time.perf_counter() - t0)
    rows = cores * rows_per_core
    flop = 4.0 * rows * SEQ * DIM
    return {"kind": kind, "cores": cores, "rows": rows, "times": times, "flop": flop,
            "sample": "%d query rows (%d per core) x all %d keys of one head; "
                      "rows are independent, so cost is linear in rows" % (rows, rows_per_core, SEQ)}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows_per_core = 32         # about a third of a second per step on each core
    for _ in range(args.warmup):
        cpu_reference_sample(rows_per_core)
    res = cpu_reference_sample(rows_per_core, repeats=args.steps)
    total = sum(res["times"])
    value = res["flop"] * args.steps / total / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "step": res["sample"]},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": res["cores"],
                         "kind": res["kind"], "sample": res["sample"]},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# Clock sampling through NVML (read-only).
# ---------------------------------------------------------------------------

class ClockSampler:
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            # CUDA ordinals follow CUDA_VISIBLE_DEVICES; NVML's do not.  Match by UUID.
            import torch
            uuid = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
            try:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _loop(self):
        n = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM))
                mask = n.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self._nvml:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# ---------------------------------------------------------------------------
# GPU arm.
# ---------------------------------------------------------------------------

SECONDARY = ("row_softmax_8192x8192", "row_softmax_1024x65536", "map_exp_8192x8192",
             "map_transpose_8192x8192", "reduce_sum_rows_8192x8192", "reduce_sum_cols_8192x8192",
             "reduce_sum_all_8192x8192", "contract_matvec_8192x8192",
             "map_chain_bias_relu_gate_8192x8192", "map_chain_shift_exp_div_8192x8192",
             "mm_t_8192x8192x4096_tf32", "mm_t_8192x8192x4096_bf16_optin",
             "mm_t_8192x8192x4096_f16_scaled", "mm_t_bias_relu_8192x8192x4096_tf32",
             "cublas_tf32_8192x8192x4096",
             "attention_16384_d128_tf32_both_contractions", "attention_16384_d128_bf16_optin")


def secondary_metrics(torch, ilang, peaks, only=None, iters=10):
    """Map / reduce / contraction figures of the other published workloads (N = 1 only).
    `only` restricts the run to one entry of SECONDARY (a short run for a profiler capture)."""
    import ctypes
    lib = ilang.core()
    vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    lib.ib_map_unary.argtypes = [ci, vp, vp, sz, vp]
    lib.ib_reduce_rows.argtypes = [ci, vp, vp, sz, sz, vp]
    lib.ib_row_softmax.argtypes = [vp, vp, sz, sz, vp]
    lib.ib_contract.argtypes = [vp, vp, vp, sz, sz, sz, sz, ci, ci, ci, vp, sz, vp]
    lib.ib_map_chain.argtypes = [ci, ctypes.POINTER(ci), ci, ctypes.POINTER(vp), ctypes.POINTER(ci),
                                 vp, sz, sz, vp]
    lib.ib_map_chain.restype = ci
    lib.ib_contract_workspace_bytes.restype = sz
    lib.ib_contract_workspace_bytes.argtypes = [sz] * 4 + [ci] * 3
    lib.ib_attention.argtypes = [vp, vp, vp, vp, sz, sz, sz, sz, sz, ci, ci, sz, vp, sz, vp]
    lib.ib_attention_workspace_bytes.argtypes = [sz, sz, sz, sz, sz, ci, ci]
    lib.ib_attention_workspace_bytes.restype = sz
    stream = torch.cuda.current_stream().cuda_stream
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device="cuda")

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        # Every iteration is queued behind a 256 MiB write that evicts L2, and the host only waits at
        # the end: the launch of iteration i is issued while the device is still writing, so the
        # interval between the two events is the device's time for fn, not the host's time to call it.
        pairs = []
        for _ in range(iters):
            flush.zero_()
            flush.zero_()                      # ~80 us of device work: covers a call through the Python front end
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            pairs.append((a, b))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in pairs) / iters

    def wanted(prefix):
        return [n for n in SECONDARY if n.startswith(prefix) and only in (None, n)]

    def hbm(nbytes, ms):
        return {"gbs": nbytes / ms / 1e6, "ms": ms, "frac_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"]}

    out = {}
    g = torch.Generator(device="cuda")
    if wanted("row_softmax_8192") or wanted("map_") or wanted("reduce_") or wanted("contract_"):
        g.manual_seed(1)
        x = 2.0 * torch.randn(8192, 8192, device="cuda", generator=g)
        y = torch.empty_like(x)
        nbytes = 2.0 * x.numel() * 4
        if wanted("row_softmax_8192"):
            out["row_softmax_8192x8192"] = hbm(nbytes, timed(
                lambda: lib.ib_row_softmax(x.data_ptr(), y.data_ptr(), 8192, 8192, stream)))
        if wanted("map_exp"):
            out["map_exp_8192x8192"] = hbm(nbytes, timed(
                lambda: lib.ib_map_unary(6, x.data_ptr(), y.data_ptr(), x.numel(), stream)))
        if wanted("reduce_sum_rows"):
            r = torch.empty(8192, device="cuda")
            out["reduce_sum_rows_8192x8192"] = hbm(x.numel() * 4.0 + 8192 * 4, timed(
                lambda: lib.ib_reduce_rows(0, x.data_ptr(), r.data_ptr(), 8192, 8192, stream)))
        if wanted("map_chain_bias"):
            # Three pointwise operators in one pass (`ij+j`, `>ij`, `ij*ij`): two full-size operands
            # and a per-column vector in, one result out.
            gate = torch.randn(8192, 8192, device="cuda", generator=g)
            bias = torch.randn(8192, device="cuda", generator=g)
            ops = (ci * 9)(0, 0, 1, 4, -2, -1, 1, -2, 2)      # add(x, bias); max(0, _); mul(_, gate)
            ptrs = (vp * 3)(x.data_ptr(), bias.data_ptr(), gate.data_ptr())
            modes = (ci * 3)(0, 2, 0)
            out["map_chain_bias_relu_gate_8192x8192"] = hbm(3.0 * x.numel() * 4 + 8192 * 4, timed(
                lambda: lib.ib_map_chain(3, ops, 3, ptrs, modes, y.data_ptr(), 8192, 8192, stream)))
            del gate
        if wanted("map_chain_shift"):
            # A softmax's two pointwise halves with the statistics supplied: `ij-i`, `^ij`, `ij/i`
            # compiled from the front end into one pointwise-chain launch.
            m = torch.randn(8192, device="cuda", generator=g)
            den = torch.rand(8192, device="cuda", generator=g) + 0.5
            chain = ilang.i("ij-i~ij") >> ilang.i("^ij~ij") >> ilang.i("ij/i~ij")
            out["map_chain_shift_exp_div_8192x8192"] = hbm(nbytes + 2 * 8192 * 4, timed(
                lambda: chain.into(y, x, m, den)))
        if wanted("reduce_sum_all"):
            # `+ij~.`: one row of 67 million columns, folded in segments.
            total = torch.empty((), device="cuda")
            fold = ilang.i("+ij~.")
            out["reduce_sum_all_8192x8192"] = hbm(x.numel() * 4.0, timed(lambda: fold.into(total, x)))
        if wanted("reduce_sum_cols"):
            # `+ij~j`: a fold of the leading axis.
            c = torch.empty(8192, device="cuda")
            fold = ilang.i("+ij~j")
            out["reduce_sum_cols_8192x8192"] = hbm(x.numel() * 4.0 + 8192 * 4, timed(lambda: fold.into(c, x)))
        if wanted("map_transpose"):
            flip = ilang.i("ij~ji")
            out["map_transpose_8192x8192"] = hbm(nbytes, timed(lambda: flip.into(y, x)))
        if wanted("contract_matvec"):
            # `ij*j~ij >> +ij~i`: a contraction with one output axis is a pass over memory.
            vec = torch.randn(8192, device="cuda", generator=g)
            r = torch.empty(8192, device="cuda")
            matvec = ilang.i("ij*j~ij") >> ilang.i("+ij~i")
            out["contract_matvec_8192x8192"] = hbm(x.numel() * 4.0 + 2 * 8192 * 4, timed(
                lambda: matvec.into(r, x, vec)))
        del x, y
    if wanted("row_softmax_1024x65536"):
        # Rows beyond one CTA's registers: held by a cluster of two.
        g.manual_seed(5)
        x = 2.0 * torch.randn(1024, 65536, device="cuda", generator=g)
        y = torch.empty_like(x)
        out["row_softmax_1024x65536"] = hbm(2.0 * x.numel() * 4, timed(
            lambda: lib.ib_row_softmax(x.data_ptr(), y.data_ptr(), 1024, 65536, stream)))
        del x, y
    if wanted("mm_t") or wanted("cublas"):
        g.manual_seed(2)
        a = 2 * torch.rand(8192, 4096, device="cuda", generator=g) - 1
        b = 2 * torch.rand(8192, 4096, device="cuda", generator=g) - 1
        c = torch.empty(8192, 8192, device="cuda")
        flop = 2.0 * 8192 * 8192 * 4096
        tf32_peak = peaks["bf16_tflops"] / 2

        def contract(precision, ws, ws_bytes):
            return timed(lambda: lib.ib_contract(a.data_ptr(), b.data_ptr(), c.data_ptr(), 1, 8192, 8192,
                                                 4096, 1, 1, precision, ws, ws_bytes, stream))

        if wanted("mm_t_8192x8192x4096_tf32"):
            ms = contract(2, None, 0)
            out["mm_t_8192x8192x4096_tf32"] = {"tflops": flop / ms / 1e9, "ms": ms,
                                               "frac_tf32_peak": flop / ms / 1e9 / tf32_peak}
        if wanted("mm_t_8192x8192x4096_bf16"):
            ws = torch.empty(2 * 8192 * 4096 * 2 + 4096, dtype=torch.uint8, device="cuda")
            ms = contract(3, ws.data_ptr(), ws.numel())
            out["mm_t_8192x8192x4096_bf16_optin"] = {
                "tflops": flop / ms / 1e9, "ms": ms, "frac_bf16_peak": flop / ms / 1e9 / peaks["bf16_tflops"],
                "note": "includes the fp32->bf16 conversion of A and B"}
        if wanted("mm_t_8192x8192x4096_f16"):
            wsf_bytes = lib.ib_contract_workspace_bytes(1, 8192, 8192, 4096, 1, 1, 5)
            wsf = torch.empty(wsf_bytes, dtype=torch.uint8, device="cuda")
            ms = contract(5, wsf.data_ptr(), wsf_bytes)
            out["mm_t_8192x8192x4096_f16_scaled"] = {
                "tflops": flop / ms / 1e9, "ms": ms, "frac_bf16_peak": flop / ms / 1e9 / peaks["bf16_tflops"],
                "frac_tf32_peak": flop / ms / 1e9 / tf32_peak,
                "note": "fp16 operands over one power of two per row (TF32's mantissa), scales restored in "
                        "the epilogue; includes the conversion of A and B"}
        if wanted("mm_t_bias_relu_8192x8192x4096_tf32"):
            # A layer, `ik*jk~ijk >> +ijk~ij >> ij+j~ij >> >ij~ij`, compiled from the front end: the bias
            # and the rectifier run in the contraction's epilogue.  Beside it the same operators as a
            # pass of their own over the stored product.
            bias = torch.randn(8192, device="cuda", generator=g)
            mm_t = (ilang.i("ik*jk~ijk") >> ilang.i("+ijk~ij")).set_precision("tf32")
            tail = ilang.i("ij+j~ij") >> ilang.i(">ij~ij")
            layer = (ilang.i("ik*jk~ijk") >> ilang.i("+ijk~ij") >> ilang.i("ij+j~ij")
                     >> ilang.i(">ij~ij")).set_precision("tf32")
            y = torch.empty_like(c)
            ms = timed(lambda: layer.into(y, a, b, bias))

            def apart():
                mm_t.into(c, a, b)
                tail.into(y, c, bias)
            ms_apart = timed(apart)
            out["mm_t_bias_relu_8192x8192x4096_tf32"] = {
                "tflops": flop / ms / 1e9, "ms": ms, "ms_as_two_passes": ms_apart,
                "note": "FLOPs of the product alone; one launch against contraction + pointwise pass"}
            del y, bias
        if wanted("cublas"):
            torch.backends.cuda.matmul.allow_tf32 = True
            ms = timed(lambda: torch.matmul(a, b.t(), out=c))
            out["cublas_tf32_8192x8192x4096"] = {"tflops": flop / ms / 1e9, "ms": ms}
        del a, b, c
    if wanted("attention"):
        # The fused attention kernel's other arms on the headline shape (one head, 16384 x 128).
        g.manual_seed(3)
        q = torch.randn(SEQ, DIM, device="cuda", generator=g) * DIM ** -0.5
        k = torch.randn(SEQ, DIM, device="cuda", generator=g)
        v = torch.randn(SEQ, DIM, device="cuda", generator=g)
        o = torch.empty_like(q)
        aflop = 4.0 * SEQ * SEQ * DIM

        def attention(precision):
            wsb = lib.ib_attention_workspace_bytes(1, SEQ, SEQ, DIM, DIM, 0, precision)
            ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
            return timed(lambda: lib.ib_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), 1,
                                                  SEQ, SEQ, DIM, DIM, 0, precision, 0, ws.data_ptr(), wsb,
                                                  stream))

        if wanted("attention_16384_d128_tf32"):
            ms = attention(2)
            out["attention_16384_d128_tf32_both_contractions"] = {
                "tflops": aflop / ms / 1e9, "ms": ms,
                "frac_tf32_peak": aflop / ms / 1e9 / (peaks["bf16_tflops"] / 2)}
        if wanted("attention_16384_d128_bf16"):
            ms = attention(3)
            out["attention_16384_d128_bf16_optin"] = {
                "tflops": aflop / ms / 1e9, "ms": ms, "frac_bf16_peak": aflop / ms / 1e9 / peaks["bf16_tflops"],
                "note": "includes the fp32->bf16 conversion of K and V"}
    return out


def multihead_block(args, torch, dist, ilang, rank, world):
    """64 heads x 32768 x 128 (the reference's multi-head case) divided over the ranks by heads
    through i_b200.sharding: every rank computes 64 / N heads in blocks and the blocks' outputs are
    assembled on every rank while the next block is computed.  Strong scaling: the work per step is
    the same at every N.  Returns the block for the JSON line (rank 0), else None."""
    import numpy as np
    from i_b200.sharding import PeerGather, sharded_attention_chunked
    heads, seq, dim = 64, 32768, DIM
    if heads % world:
        return {"unavailable": "64 heads do not divide over %d ranks" % world}
    per = heads // world
    g = torch.Generator(device="cuda")
    g.manual_seed(4 + rank)
    q = torch.randn(per, seq, dim, device="cuda", generator=g) * dim ** -0.5
    k = torch.randn(per, seq, dim, device="cuda", generator=g)
    v = torch.randn(per, seq, dim, device="cuda", generator=g)
    attn = readme_attention(ilang, batched=True).set_precision(args.precision)
    flop = heads * 4.0 * seq * seq * dim
    chunks = min(per, 4)
    main = torch.cuda.current_stream()
    steps, warm = 4, 2

    def attend_into(o, qs, ks, vs):
        attn.into(o, qs, ks, vs)

    def timed(run, finish=None):
        for _ in range(warm):
            run()
        if finish:
            finish()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(main)
        for _ in range(steps):
            run()
        b.record(main)
        torch.cuda.synchronize()
        if finish:
            finish()
        ms = a.elapsed_time(b)
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        ms /= steps
        return {"value": flop / ms / 1e9, "unit": "TFLOP/s", "ms_per_step": ms}

    out = {"workload": "64 heads x seq 32768 x d 128, fp32 N(0,1) seeds 4 + rank (generated on the "
                       "device), Q * 1/sqrt(128); %d heads per rank in %d blocks" % (per, chunks),
           "scaling": "strong", "steps": steps, "warmup": warm}
    own = torch.empty(per, seq, dim, device="cuda")

    def compute_only():
        for c in range(chunks):
            lo, hi = c * per // chunks, (c + 1) * per // chunks
            attend_into(own[lo:hi], q[lo:hi], k[lo:hi], v[lo:hi])

    out["assembly_off"] = timed(compute_only)
    check = own
    if world > 1:
        # (a) copy engines into peer-mapped buffers, block by block under the next block's kernel.
        if args.gather in ("auto", "ce") and PeerGather.available():
            try:
                peer = PeerGather((per, seq, dim), slots=2)
            except Exception as exc:                      # noqa: BLE001
                peer = None
                out["copy_engine"] = {"unavailable": str(exc)[:200]}
            ok = torch.tensor([1 if peer is not None else 0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 1:
                state = {"n": 0}

                def run_ce():
                    slot = state["n"] % 2
                    state["n"] += 1
                    peer.wait_on(main, peer.reusable(slot))
                    sharded_attention_chunked(attend_into, q, k, v, None, chunks=chunks, gather=peer,
                                              slot=slot, local_inputs=True)

                def finish_ce():
                    peer.join(main)
                    peer.finish()

                out["copy_engine"] = timed(run_ce, finish_ce)
                full = peer.gathered((state["n"] - 1) % 2)
                mine = full[rank].contiguous().view(torch.int32).to(torch.int64).sum().reshape(1)
                owners = torch.empty(world, dtype=torch.int64, device="cuda")
                dist.all_gather_into_tensor(owners, mine)
                seen = full.contiguous().view(torch.int32).to(torch.int64).reshape(world, -1).sum(dim=1)
                good = torch.tensor([1 if torch.equal(seen, owners) else 0], device="cuda")
                dist.all_reduce(good, op=dist.ReduceOp.MIN)
                out["copy_engine"]["gathered_output_verified"] = bool(good.item())
                check = full[rank]
                del peer, full
        # (b) NCCL all-gather per block on a side stream, a few SMs kept free for its kernels.
        if args.gather in ("auto", "nccl"):
            whole = torch.empty(heads, seq, dim, device="cuda")
            ilang.set_reserved_sms(args.reserve_sms)

            def run_nccl():
                sharded_attention_chunked(attend_into, q, k, v, whole, chunks=chunks, local_inputs=True)

            out["nccl"] = timed(run_nccl)
            out["nccl"]["reserved_sms"] = args.reserve_sms
            ilang.set_reserved_sms(0)
            del whole
        headline = out.get("copy_engine") if "value" in out.get("copy_engine", {}) else out.get("nccl")
    else:
        headline = out["assembly_off"]
    if headline and "value" in headline:
        out["value"], out["ms_per_step"], out["unit"] = headline["value"], headline["ms_per_step"], "TFLOP/s"
    if rank != 0:
        return None
    # 64 rows of this rank's first head against the CPU reference.
    import oracle
    rows = (np.arange(64) * 512 + (129 * np.arange(64)) % 512).astype(np.int64)
    q0, k0, v0 = q[0].cpu().numpy(), k[0].cpu().numpy(), v[0].cpu().numpy()
    ref_fn = oracle.reference_attention if oracle.have_reference() else oracle.attention_fused
    cores = os.cpu_count() or 1
    cuts = np.linspace(0, rows.size, min(cores, rows.size) + 1).astype(int)
    ref = np.concatenate(oracle.reference_attention_rows(
        q0[rows], k0, v0, [(a, b) for a, b in zip(cuts[:-1], cuts[1:]) if b > a], threads=cores, fn=ref_fn))
    got = check[0][torch.from_numpy(rows).cuda()].cpu().numpy()
    out["parity_max_rel_to_peak_vs_oracle"] = float(np.abs(got - ref).max() / np.abs(ref).max())
    out["parity_rows"] = int(rows.size)
    return out


def run_gpu_arm(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the hot path has no CPU fallback)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from i_b200 import build as lib_build
    if not os.path.exists(lib_build.LIB):
        lib_build.build()
    from i_b200 import ilang

    peaks = load_peaks()
    if args.only:
        if world > 1:
            raise SystemExit("--only is a single-GPU run")
        res = secondary_metrics(torch, ilang, peaks, only=args.only, iters=max(1, args.steps))
        print(json.dumps({"only": args.only, "iters": max(1, args.steps), "result": res.get(args.only)}),
              flush=True)
        return
    heads = args.heads
    batched = heads > 1
    # "auto" is what a caller gets without asking: for attention of this size the arm that runs
    # both contractions on fp16 operands stored over powers of two (10-bit mantissa, like TF32).
    attn = readme_attention(ilang, batched=batched).set_precision(args.precision)
    flop_per_step = heads * FLOP_PER_HEAD

    def shaped(t):
        return t if batched else t[0]

    # Distinct input sets per rank (seed 3 for set 0 of rank 0, the published case's seed);
    # enough of them that one pass over all sets exceeds L2.
    set_bytes = 4 * heads * SEQ * DIM * 4
    rotation = max(2, min(ROTATION, -(-256 * 1024 * 1024 // set_bytes)))
    sets = []
    for s in range(rotation):
        q, k, v = make_inputs(seed=3 + 1000 * rank + s, heads=heads)
        sets.append(tuple(shaped(torch.from_numpy(t)).cuda() for t in (q, k, v)))
    out_shape = (heads, SEQ, DIM) if batched else (SEQ, DIM)
    main = torch.cuda.current_stream()
    computed = torch.cuda.Event()

    # Output assembly at N > 1.  Preferred: copy engines over NVLink into peer-mapped
    # buffers (no SM is taken from the persistent attention kernel).  Fallback: NCCL
    # all-gather on a side stream with a few SMs reserved for its kernels.
    gather_mode = "none"
    peer = None
    if world > 1:
        from i_b200.sharding import PeerGather
        want_ce = args.gather in ("auto", "ce") and PeerGather.available()
        ok = torch.tensor([1 if want_ce else 0], device="cuda")
        if want_ce:
            try:
                peer = PeerGather(out_shape, slots=2)
            except Exception as exc:                      # noqa: BLE001
                if rank == 0:
                    sys.stderr.write("peer-mapped gather unavailable (%s); using NCCL\n" % exc)
                ok[0] = 0
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 1:
            gather_mode = "copy-engine peer writes"
        else:
            peer = None
            gather_mode = "nccl all_gather_into_tensor, %d SMs reserved" % args.reserve_sms
            ilang.set_reserved_sms(args.reserve_sms)
    if peer is not None:
        outs = [peer.local(0), peer.local(1)]
        gathered = None
        side = None
    else:
        gathered = [torch.empty((world,) + out_shape, device="cuda") for _ in range(2)]
        outs = [g[rank] for g in gathered]
        side = torch.cuda.Stream() if world > 1 else None
    gather_done = [None, None]

    def step(s):
        q, k, v = sets[s % rotation]
        buf = s % 2
        if gather_done[buf] is not None:           # the gather of step s-2 still reads this buffer
            if peer is not None:
                peer.wait_on(main, gather_done[buf])
            else:
                main.wait_event(gather_done[buf])
        attn.into(outs[buf], q, k, v)
        if peer is not None:
            computed.record(main)
            gather_done[buf] = peer.publish(buf, computed)
        elif side is not None:
            computed.record(main)
            side.wait_event(computed)
            with torch.cuda.stream(side):
                dist.all_gather_into_tensor(gathered[buf].view(-1), outs[buf].reshape(-1))
                gather_done[buf] = torch.cuda.Event()
                gather_done[buf].record(side)

    for s in range(max(args.warmup, 3)):
        step(s)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    launches0 = ilang.launch_count()
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin.record(main)
    for s in range(args.steps):
        step(s)
    if peer is not None:
        peer.join(main)
    elif side is not None:
        main.wait_stream(side)
    t_end.record(main)
    torch.cuda.synchronize()
    launches = ilang.launch_count() - launches0
    elapsed_ms = t_begin.elapsed_time(t_end)
    gather_ok = None
    if peer is not None:
        peer.finish()
    if world > 1:
        # Every rank must now hold every rank's output of the last step: compare a
        # checksum of each gathered row with the checksum its owner computed.
        last = (args.steps - 1) % 2
        full = peer.gathered(last) if peer is not None else gathered[last]
        torch.cuda.synchronize()
        # Integer sums of the raw bits: exact whatever the reduction order.
        mine = outs[last].contiguous().view(torch.int32).to(torch.int64).sum().reshape(1)
        owners = torch.empty(world, dtype=torch.int64, device="cuda")
        dist.all_gather_into_tensor(owners, mine)
        seen = full.contiguous().view(torch.int32).to(torch.int64).reshape(world, -1).sum(dim=1)
        good = torch.tensor([1 if torch.equal(seen, owners) else 0], device="cuda")
        dist.all_reduce(good, op=dist.ReduceOp.MIN)
        gather_ok = bool(good.item())
        dist.barrier()
        t = torch.tensor([elapsed_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = world * flop_per_step / ms_per_step / 1e9

    if args.kernel_only:
        sampler.stop()
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world,
                              "steps": args.steps, "ms_per_step": ms_per_step, "heads": heads,
                              "seq": SEQ, "note": "kernel-only run for profiling"}), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # The same loop for about two seconds: the figure a long-running job sees under the power cap.
    sustained = None
    if not args.no_sustained:
        n_long = max(args.steps, min(20000, int(2000.0 / ms_per_step)))
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s_begin, s_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_begin.record(main)
        for s in range(n_long):
            step(s)
        if peer is not None:
            peer.join(main)
        elif side is not None:
            main.wait_stream(side)
        s_end.record(main)
        torch.cuda.synchronize()
        long_ms = s_begin.elapsed_time(s_end)
        if peer is not None:
            peer.finish()
        if world > 1:
            t = torch.tensor([long_ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            long_ms = float(t.item())
        sustained = {"value": world * flop_per_step * n_long / long_ms / 1e9, "unit": "TFLOP/s",
                     "steps": n_long, "seconds": long_ms / 1e3, "ms_per_step": long_ms / n_long}

    multi = None
    if not args.no_multihead and heads == 1 and SEQ == 16384:
        multi = multihead_block(args, torch, dist, ilang, rank, world)

    # End to end through the host-pointer C ABI (i_exec_into), pinned host buffers.
    hq, hk, hv = (shaped(torch.from_numpy(t)).pin_memory()
                  for t in make_inputs(seed=3 + 1000 * rank, heads=heads))
    ho = torch.empty(out_shape).pin_memory()
    nq, nk, nv, no = (t.numpy() for t in (hq, hk, hv, ho))
    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(2):
        attn.into(no, nq, nk, nv)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        attn.into(no, nq, nk, nv)              # returns when O is back in host memory
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    sampler.stop()
    e2e_value = world * flop_per_step * e2e_steps / e2e_s / 1e12

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # Parity spot check of the timed kernel (never timed): 1024 rows, eight in every 128-row tile
    # at offsets that differ from tile to tile, against the reference's own emitted C on all host
    # cores (the restated loop nest when that library is absent).
    import oracle
    q0, k0, v0 = (t.cpu().numpy().reshape(-1, SEQ, DIM)[0] for t in sets[0])
    got = attn.exec_torch(*sets[0]).cpu().numpy().reshape(-1, SEQ, DIM)[0]
    tiles = np.arange(SEQ // 128)
    rows = np.sort(np.concatenate([tiles * 128 + (17 * j + 5 * tiles) % 128 for j in range(8)]))
    ref_fn = oracle.reference_attention if oracle.have_reference() else oracle.attention_fused
    cores = os.cpu_count() or 1
    cuts = np.linspace(0, rows.size, min(cores, rows.size) + 1).astype(int)
    ref = np.concatenate(oracle.reference_attention_rows(
        q0[rows], k0, v0, [(a, b) for a, b in zip(cuts[:-1], cuts[1:]) if b > a], threads=cores, fn=ref_fn))
    parity = float(np.abs(got[rows] - ref).max() / np.abs(ref).max())

    tf32_peak = peaks["bf16_tflops"] / 2.0
    f16_peak = peaks["bf16_tflops"]            # fp16 and bf16 issue at the same rate
    f16_arm = args.precision in ("auto", "f16")
    mixed = args.precision == "tf32_f16"
    if args.precision == "bf16":
        arm_peak, arm_dtype = f16_peak, "bf16"
        arm_text = "tcgen05 kind::f16 on bf16 operands, fp32 accumulate"
        peak_text = "%s bf16_tflops %.1f" % (peaks["source"], peaks["bf16_tflops"])
    elif f16_arm:
        arm_peak, arm_dtype = f16_peak, "f16"
        arm_text = ("both contractions tcgen05 kind::f16 on fp16 operands (10-bit mantissa like TF32): "
                    "Q per query row, K per 128-key tile and V per head stored over powers of two "
                    "that bring them into fp16's range, scales restored exactly in fp32; fp32 "
                    "accumulate, fp32 softmax statistics")
        peak_text = ("%s bf16_tflops %.1f (fp16 and bf16 issue at the same rate)"
                     % (peaks["source"], peaks["bf16_tflops"]))
    elif mixed:
        # Half of the FLOPs (Q K^T) run at the TF32 rate, half (P V) at the 16-bit rate.
        arm_peak, arm_dtype = 2.0 / (1.0 / tf32_peak + 1.0 / f16_peak), "tf32+f16"
        arm_text = ("S = Q K^T: tcgen05 kind::tf32; O += P V: kind::f16 on fp16 operands (10-bit "
                    "mantissa like TF32, V scaled per head by a power of two); fp32 accumulate")
        peak_text = ("%s bf16_tflops %.1f: half the FLOPs at the TF32 rate (bf16 / 2), half at the "
                     "16-bit rate -> harmonic mean" % (peaks["source"], peaks["bf16_tflops"]))
    else:
        arm_peak, arm_dtype = tf32_peak, "tf32"
        arm_text = "tcgen05 kind::tf32 for both contractions, fp32 accumulate"
        peak_text = ("%s bf16_tflops %.1f / 2 (TF32 MMA issues at half the bf16 rate)"
                     % (peaks["source"], peaks["bf16_tflops"]))
    achieved = flop_per_step / ms_per_step / 1e9
    traffic = ATTENTION_DRAM_BYTES_PER_LAUNCH.get(arm_dtype) if (heads == 1 and SEQ == 16384) else None
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": arm_dtype, "data": "synthetic",
        "config": {"workload": WORKLOAD if (heads == 1 and SEQ == 16384) else
                   "%d heads x seq %d x d %d per rank per step (batched README attention)"
                   % (heads, SEQ, DIM),
                   "units_per_rank_per_step": heads,
                   "l2": "inputs rotate over %d distinct sets (%d MiB) > 126 MB L2"
                         % (rotation, rotation * set_bytes // 2 ** 20),
                   "multi_gpu": "one head per rank per step; output assembly: " + gather_mode,
                   "gathered_output_verified": gather_ok,
                   "precision": arm_text,
                   "parity_max_rel_to_peak_vs_oracle": parity,
                   "parity_rows": int(rows.size),
                   "parity_against": "reference's emitted C (oracle/_ref)" if oracle.have_reference()
                   else "restated loop nest (oracle)"},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": arm_peak, "unit": "TFLOP/s",
                     "frac": achieved / arm_peak, "traffic": traffic,
                     "peak_source": peak_text,
                     "frac_of_tf32_peak": achieved / tf32_peak,
                     "frac_of_bf16_peak": achieved / peaks["bf16_tflops"],
                     "note": "achieved = 4*Nq*Nk*d FLOP / average step time on one rank; a step "
                             "launches the operand-preparation, attention and merge kernels"},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s",
                "h2d_bytes_per_step": 3 * heads * SEQ * DIM * 4,
                "d2h_bytes_per_step": heads * SEQ * DIM * 4, "steps": e2e_steps},
        "gpu_launches": launches,
        "clocks": sampler.summary(),
    }
    if sustained is not None:
        line["sustained"] = sustained
    if multi is not None:
        line["heads64_seq32768"] = multi
    if world == 1 and f16_arm:
        # The same steps on the arms that keep TF32 operands, for comparison in the same run.
        for key, prec, note in (
                ("tf32_both_contractions", "tf32",
                 "same workload and loop with --precision tf32 (Q K^T and P V both kind::tf32)"),
                ("tf32_logits_f16_values", "tf32_f16",
                 "same workload and loop with --precision tf32_f16 (Q K^T kind::tf32, P V kind::f16)")):
            other = readme_attention(ilang, batched=batched).set_precision(prec)
            for s2 in range(3):
                other.into(outs[s2 % 2], *sets[s2 % rotation])
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(main)
            for s2 in range(args.steps):
                other.into(outs[s2 % 2], *sets[s2 % rotation])
            b.record(main)
            torch.cuda.synchronize()
            other_ms = a.elapsed_time(b) / args.steps
            other_tf = flop_per_step / other_ms / 1e9
            line[key] = {"value": other_tf, "unit": "TFLOP/s", "ms_per_step": other_ms,
                         "frac_of_tf32_peak": other_tf / tf32_peak, "note": note}
    if world == 1:
        res = cpu_reference_sample(256)        # ~20 s of CPU work over all cores
        line["cpu_baseline"] = {"value": res["flop"] / res["times"][0] / 1e12, "unit": "TFLOP/s",
                                "cores": res["cores"], "kind": res["kind"], "sample": res["sample"]}
        if not args.no_secondary and heads == 1 and SEQ == 16384:
            line["secondary"] = secondary_metrics(torch, ilang, peaks)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default=None, choices=SECONDARY,
                    help="run one side measurement alone, --steps iterations of it (N = 1)")
    ap.add_argument("--no-sustained", action="store_true", help="skip the two-second loop")
    ap.add_argument("--no-multihead", action="store_true",
                    help="skip the 64-head x 32768 block (sharded over the ranks)")
    ap.add_argument("--no-secondary", action="store_true",
                    help="skip the map/reduce/contraction side measurements")
    ap.add_argument("--kernel-only", action="store_true",
                    help="device-timed loop only (no end-to-end, CPU or side measurements); "
                         "for profiler captures")
    ap.add_argument("--gather", default="auto", choices=["auto", "ce", "nccl"],
                    help="output assembly at N > 1: copy-engine peer writes or NCCL all-gather")
    ap.add_argument("--reserve-sms", type=int, default=20,
                    help="SMs left free for NCCL kernels when the NCCL gather is used")
    ap.add_argument("--precision", default="auto", choices=["auto", "tf32", "bf16", "tf32_f16", "f16"],
                    help="arithmetic of the fused attention kernel (default: the library's own choice)")
    ap.add_argument("--heads", type=int, default=1,
                    help="heads per rank per step (default 1, the headline case)")
    ap.add_argument("--seq", type=int, default=16384, help="sequence length (default 16384)")
    args = ap.parse_args()
    global SEQ, FLOP_PER_HEAD
    SEQ = args.seq
    FLOP_PER_HEAD = 4.0 * SEQ * SEQ * DIM
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
