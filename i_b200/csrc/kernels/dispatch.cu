// ib_contract and ib_attention: precision choice, workspace carving and the
// layout fix-ups that give the tensor-core kernels K-major operands.
#include <initializer_list>
#include "common.cuh"
#include "kernels.h"

namespace ib {
namespace {

constexpr double kTensorMinFlop = 268435456.0;  // 2^28: below this the fp32 arm is used

size_t round_up(size_t x, size_t to) { return (x + to - 1) / to * to; }

// Sub-allocator over the caller's workspace (256-byte granules).
// Largest element count whose byte size, rounded up and summed a few times, stays inside size_t.
constexpr size_t kMaxFloats = SIZE_MAX >> 6;

// True when the product of the extents does not fit kMaxFloats (or overflows on the way).
bool too_many_elements(std::initializer_list<size_t> extents) {
  size_t product = 1;
  for (size_t e : extents)
    if (__builtin_mul_overflow(product, e, &product)) return true;
  return product > kMaxFloats;
}

struct Carver {
  uint8_t* base;
  size_t size, used = 0;
  Carver(void* p, size_t n) : base(static_cast<uint8_t*>(p)), size(n) {}
  float* take(size_t floats) {
    if (floats > kMaxFloats) return nullptr;
    size_t bytes = round_up(floats * sizeof(float), 256);
    if (!base || bytes > size || used > size - bytes) return nullptr;
    float* out = reinterpret_cast<float*>(base + used);
    used += bytes;
    return out;
  }
};

size_t carve_bytes(size_t floats) {
  return floats > kMaxFloats ? SIZE_MAX >> 4 : round_up(floats * sizeof(float), 256);
}

// Parts into which the k range of a contraction with few output tiles is cut, so that every SM
// has work: an output of 128 x 128 is four tiles of the fp32 arm (one of the tensor arm), and a
// k of thousands would run on that many SMs.  Each part sums into its own copy of the result
// and the copies are added.  `tile`: output rows and columns per CTA of the arm.  1 = whole.
size_t k_parts(size_t batch, size_t m, size_t n, size_t k, size_t tile) {
  const size_t tiles = batch * ((m + tile - 1) / tile) * ((n + tile - 1) / tile);
  if (tiles == 0 || tiles * 2 > static_cast<size_t>(kNumSMs) || k < 1024) return 1;
  size_t parts = static_cast<size_t>(kNumSMs) * 2 / tiles;
  if (parts > k / 128) parts = k / 128;
  if (parts > 64) parts = 64;
  if (batch * parts > 65535) parts = 65535 / batch;
  return parts < 2 ? 1 : parts;
}

// The same for the TF32 tensor arm, which takes the parts as batch entries of one tensor map:
// one batch entry only, and parts of equal length, a multiple of four.
size_t k_parts_tensor(size_t batch, size_t m, size_t n, size_t k) {
  if (batch != 1) return 1;
  for (size_t parts = k_parts(1, m, n, k, 128); parts >= 2; --parts)
    if (k % (4 * parts) == 0) return parts;
  return 1;
}

bool wants_tensor(int precision, double flop) {
  if (precision == IB_PRECISION_FP32) return false;
  if (precision == IB_PRECISION_AUTO) return flop >= kTensorMinFlop;
  return true;
}

// AUTO takes the fp16 arm for a contraction only where its two conversion passes (each operand
// read twice and written once at half size) are paid back by the faster MMAs: both output extents
// large against the operand sizes and a deep contraction.  Measured on B200: 8192 x 8192 x 4096 runs
// 1.58x faster than the TF32 arm, 8192 x 8192 x 512 and 16384 x 128 x 16384 slower.
bool contract_prefers_f16(size_t m, size_t n, size_t k) {
  return k >= 2048 && m >= 4096 && n >= 4096;
}

// Shape-only test (no pointers): can the tensor arm take this contraction?
bool contract_shape_ok(size_t k) { return k % 4 == 0 && k >= 4; }

bool attention_shape_ok(size_t d, size_t dv) {
  return d % 4 == 0 && d >= 4 && d <= 128 && dv >= 1 && dv <= 128;
}

// Which arithmetic the fused attention kernel uses for a precision request: AUTO and F16 take the
// fp16 arm (both contractions on fp16 operands scaled into range: TF32's mantissa, half the
// tensor-core instructions), TF32_F16 the mixed arm (TF32 for Q K^T, fp16 for P V), TF32 the pure
// TF32 arm, BF16 the bf16 arm.
AttentionArm attention_arm(int precision) {
  if (precision == IB_PRECISION_BF16) return AttentionArm::BF16;
  if (precision == IB_PRECISION_TF32) return AttentionArm::TF32;
  if (precision == IB_PRECISION_TF32_F16) return AttentionArm::MIXED;
  return AttentionArm::F16;
}

// The attention kernel's K and V operands: rounded (TF32), converted (BF16) or mixed copies,
// V transposed to [dv][keys]; the mixed arm also keeps one scale per head.
struct PreparedKV {
  const void* k = nullptr;
  const void* vt = nullptr;
  const float* v_scale = nullptr;
  const float* k_tile_scale = nullptr;
  size_t d_pitch = 0, nk_pitch = 0;
  AttentionArm arm = AttentionArm::TF32;
};

size_t prepared_kv_bytes(size_t batch, size_t nk, size_t d, size_t dv, AttentionArm arm) {
  if (arm == AttentionArm::BF16)
    return carve_bytes((batch * nk * round_up(d, 8) + 1) / 2) +
           carve_bytes((batch * dv * round_up(nk, 8) + 1) / 2);
  if (arm == AttentionArm::F16)
    return carve_bytes((batch * nk * round_up(d, 8) + 1) / 2) +
           carve_bytes((batch * dv * round_up(nk, 8) + 1) / 2) + carve_bytes(batch) +
           carve_bytes(batch * kAbsmaxBlocks) + carve_bytes(batch * ((nk + 127) / 128));
  if (arm == AttentionArm::MIXED)
    return carve_bytes(batch * nk * d) + carve_bytes((batch * dv * round_up(nk, 8) + 1) / 2) +
           carve_bytes(batch) + carve_bytes(batch * kAbsmaxBlocks);
  return carve_bytes(batch * nk * d) + carve_bytes(batch * dv * round_up(nk, 4));
}

// Carves the copies out of `ws`; with `fill` it also launches the kernels that write them.
int prepared_kv(const float* k, const float* v, size_t batch, size_t nk, size_t d, size_t dv,
                bool v_kmajor, AttentionArm arm, bool fill, Carver& ws, PreparedKV* out,
                cudaStream_t s) {
  const char* small = "ib_attention: workspace too small (see the matching *_bytes function)";
  out->arm = arm;
  if (arm == AttentionArm::BF16) {
    // Opt-in: bf16 operands (round to nearest even), fp32 scores, sums and outputs.
    out->d_pitch = round_up(d, 8);
    out->nk_pitch = round_up(nk, 8);
    float* k16 = ws.take((batch * nk * out->d_pitch + 1) / 2);
    float* vt16 = ws.take((batch * dv * out->nk_pitch + 1) / 2);
    if (!k16 || !vt16) return fail(small);
    out->k = k16;
    out->vt = vt16;
    if (!fill) return 0;
    return prepare_attention_operands_bf16(k, k16, v, vt16, batch, nk, d, dv, out->d_pitch,
                                           out->nk_pitch, v_kmajor, s);
  }
  if (arm == AttentionArm::F16) {
    // Both operands fp16: K over one power of two per tile of 128 keys, V^T over one per head.
    out->d_pitch = round_up(d, 8);
    out->nk_pitch = round_up(nk, 8);
    float* k16 = ws.take((batch * nk * out->d_pitch + 1) / 2);
    float* vt16 = ws.take((batch * dv * out->nk_pitch + 1) / 2);
    float* scale = ws.take(batch);
    float* block_max = ws.take(batch * kAbsmaxBlocks);
    float* k_tile_scale = ws.take(batch * ((nk + 127) / 128));
    if (!k16 || !vt16 || !scale || !block_max || !k_tile_scale) return fail(small);
    out->k = k16;
    out->vt = vt16;
    out->v_scale = scale;
    out->k_tile_scale = k_tile_scale;
    if (!fill) return 0;
    return prepare_attention_operands_f16(k, k16, k_tile_scale, v, vt16, scale, block_max, batch, nk,
                                          d, dv, out->d_pitch, out->nk_pitch, v_kmajor, s);
  }
  if (arm == AttentionArm::MIXED) {
    // K rounded to TF32; V^T as fp16 of V / scale[head], the scale a power of two that brings
    // the head's largest magnitude into [2^14, 2^15).
    out->d_pitch = d;
    out->nk_pitch = round_up(nk, 8);
    float* kr = ws.take(batch * nk * d);
    float* vt16 = ws.take((batch * dv * out->nk_pitch + 1) / 2);
    float* scale = ws.take(batch);
    float* block_max = ws.take(batch * kAbsmaxBlocks);
    if (!kr || !vt16 || !scale || !block_max) return fail(small);
    out->k = kr;
    out->vt = vt16;
    out->v_scale = scale;
    if (!fill) return 0;
    return prepare_attention_operands_mixed(k, kr, v, vt16, scale, block_max, batch, nk, d, dv,
                                            out->nk_pitch, v_kmajor, s);
  }
  // Pure TF32.  The tensor core truncates fp32 operands to TF32, so K and V are first rounded
  // to nearest into workspace copies (V transposed to [dv][keys] on the way, the K-major
  // layout the second contraction needs); the kernel rounds Q itself while moving it into
  // tensor memory.
  out->d_pitch = d;
  out->nk_pitch = round_up(nk, 4);
  float* kr = ws.take(batch * nk * d);
  float* vt = ws.take(batch * dv * out->nk_pitch);
  if (!kr || !vt) return fail(small);
  out->k = kr;
  out->vt = vt;
  if (!fill) return 0;
  const bool aligned = (reinterpret_cast<uintptr_t>(k) & 15u) == 0;
  if (!v_kmajor && aligned)
    return prepare_attention_operands(nullptr, nullptr, 0, k, kr, batch * nk * d, v, vt, batch, nk,
                                      dv, out->nk_pitch, s);
  if (int rc = round_tf32_rows(k, kr, batch * nk, d, d, d, nullptr, nullptr, 0, 0, 0, 0, s)) return rc;
  if (!v_kmajor) return transpose_batched(v, vt, batch, nk, dv, out->nk_pitch, true, s);
  return round_tf32_rows(v, vt, batch * dv, nk, nk, out->nk_pitch, nullptr, nullptr, 0, 0, 0, 0, s);
}

}  // namespace
}  // namespace ib

extern "C" size_t ib_contract_workspace_bytes(size_t batch, size_t m, size_t n, size_t k,
                                              int a_kmajor, int b_kmajor, int precision) {
  using namespace ib;
  // Extents whose element counts do not fit size_t: no workspace can serve them (ib_contract
  // refuses the same extents).
  if (too_many_elements({batch, m, k}) || too_many_elements({batch, n, k}) ||
      too_many_elements({batch, m, n}))
    return SIZE_MAX;
  if (precision == IB_PRECISION_TF32_F16) precision = IB_PRECISION_TF32;   // attention-only distinction
  // Vector times a matrix stored [k][columns]: the slabs' partial sums of the fold down its columns.
  if (m != 1 || n != 1) {
    constexpr size_t kMostLaunches = 64;      // as in the contraction itself
    if (batch <= kMostLaunches) {
      if (n == 1) return a_kmajor ? 0 : carve_bytes(dot_leading_axis_floats(k, m));
      if (m == 1) return b_kmajor ? 0 : carve_bytes(dot_leading_axis_floats(k, n));
    }
  } else {
    return carve_bytes(long_rows_floats(batch, k));   // dot products of few, very long rows
  }
  const double flop = 2.0 * batch * m * n * k;
  // Copies of the result when the k range is cut into parts (either 32-bit arm).
  const size_t parts = std::max(k_parts(batch, m, n, k, 64), k_parts_tensor(batch, m, n, k));
  const size_t copies = parts > 1 ? carve_bytes(batch * parts * m * n) : 0;
  if (!wants_tensor(precision, flop)) return copies;
  if (precision == IB_PRECISION_AUTO && contract_prefers_f16(m, n, k)) precision = IB_PRECISION_F16;
  if (precision == IB_PRECISION_F16) {
    // fp16 copies of both operands plus one scale per row; fp32 transposes first when needed.
    const size_t kp = round_up(k, 8);
    size_t bytes = carve_bytes((batch * m * kp + 1) / 2) + carve_bytes((batch * n * kp + 1) / 2) +
                   carve_bytes(batch * m) + carve_bytes(batch * n);
    if (!a_kmajor) bytes += carve_bytes(batch * m * k);
    if (!b_kmajor) bytes += carve_bytes(batch * n * k);
    return bytes;
  }
  if (precision == IB_PRECISION_BF16) {
    // bf16 copies of both operands ([rows][k rounded up to 8]); fp32 transposes first when needed.
    const size_t kp = round_up(k, 8);
    size_t bytes = carve_bytes((batch * m * kp + 1) / 2) + carve_bytes((batch * n * kp + 1) / 2);
    if (!a_kmajor) bytes += carve_bytes(batch * m * k);
    if (!b_kmajor) bytes += carve_bytes(batch * n * k);
    return bytes;
  }
  if (!contract_shape_ok(k)) return copies;
  size_t bytes = copies;
  if (!a_kmajor) bytes += carve_bytes(batch * m * k);
  if (!b_kmajor) bytes += carve_bytes(batch * n * k);
  return bytes;
}

extern "C" int ib_transpose(const float* x, float* y, size_t batch, size_t rows, size_t cols,
                            void* stream) {
  using namespace ib;
  if (batch == 0 || rows == 0 || cols == 0) return 0;
  if (!x || !y) return fail("ib_transpose: null pointer");
  if (too_many_elements({batch, rows, cols})) return fail("ib_transpose: extents too large");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The tile kernel takes up to 65535 batch entries and row tiles per launch.
  constexpr size_t kMost = 65535;
  if ((rows + 63) / 64 > kMost) return fail("ib_transpose: more than 4194240 rows");
  for (size_t b0 = 0; b0 < batch; b0 += kMost) {
    const size_t nb = batch - b0 < kMost ? batch - b0 : kMost;
    if (int rc = transpose_batched(x + b0 * rows * cols, y + b0 * rows * cols, nb, rows, cols, rows, false, s))
      return rc;
  }
  return 0;
}

extern "C" int ib_contract(const float* a, const float* b, float* c, size_t batch, size_t m,
                           size_t n, size_t k, int a_kmajor, int b_kmajor, int precision,
                           void* workspace, size_t workspace_bytes, void* stream) {
  return ib_contract_tiled(a, b, c, batch, m, n, k, a_kmajor, b_kmajor, precision, 0, 0, workspace,
                           workspace_bytes, stream);
}

namespace ib {
namespace {

// Pointwise operators that follow a contraction, in the two forms its arms need: `fused` for the
// tensor-core kernels' epilogue, and the same list as an ib_map_chain call over the stored result
// for the arms that have no epilogue hook (fp32, and a contraction over no terms).
struct ContractChain {
  GemmEpilogue fused;
  int n_ops = 0;
  int ops[3 * IB_MAX_CHAIN_OPS] = {};
  int n_operands = 0;                       // of the ib_map_chain form: the result first
  const float* operands[IB_MAX_CHAIN_OPERANDS] = {};
  int modes[IB_MAX_CHAIN_OPERANDS] = {};

  int in_place(float* c, size_t rows, size_t cols, void* stream) const {
    if (n_ops == 0) return 0;
    const float* list[IB_MAX_CHAIN_OPERANDS];
    for (int i = 0; i < n_operands; ++i) list[i] = i == 0 ? c : operands[i];
    return ib_map_chain(n_ops, ops, n_operands, list, modes, c, rows, cols, stream);
  }
};

int contract_with_chain(const float* a, const float* b, float* c, size_t batch, size_t m, size_t n,
                        size_t k, int a_kmajor, int b_kmajor, int precision, size_t col_tile,
                        size_t col_group, const ContractChain* chain, void* workspace,
                        size_t workspace_bytes, void* stream);

}  // namespace
}  // namespace ib

extern "C" int ib_contract_tiled(const float* a, const float* b, float* c, size_t batch, size_t m,
                                 size_t n, size_t k, int a_kmajor, int b_kmajor, int precision,
                                 size_t col_tile, size_t col_group, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  return ib::contract_with_chain(a, b, c, batch, m, n, k, a_kmajor, b_kmajor, precision, col_tile,
                                 col_group, nullptr, workspace, workspace_bytes, stream);
}

extern "C" int ib_contract_chain(const float* a, const float* b, float* c, size_t batch, size_t m,
                                 size_t n, size_t k, int a_kmajor, int b_kmajor, int precision,
                                 size_t col_tile, size_t col_group, int n_ops, const int* ops,
                                 int n_operands, const float* const* operands, const int* modes,
                                 void* workspace, size_t workspace_bytes, void* stream) {
  using namespace ib;
  if (n_ops == 0)
    return contract_with_chain(a, b, c, batch, m, n, k, a_kmajor, b_kmajor, precision, col_tile,
                               col_group, nullptr, workspace, workspace_bytes, stream);
  if (n_ops < 0 || n_ops > IB_MAX_CHAIN_OPS || !ops)
    return fail("ib_contract_chain: between 0 and " + std::to_string(IB_MAX_CHAIN_OPS) + " operators");
  if (n_operands < 0 || n_operands > IB_MAX_CHAIN_OPERANDS - 1 || (n_operands > 0 && (!operands || !modes)))
    return fail("ib_contract_chain: at most " + std::to_string(IB_MAX_CHAIN_OPERANDS - 1) +
                " operands beside the contraction");
  ContractChain chain;
  chain.n_ops = n_ops;
  chain.n_operands = n_operands + 1;
  chain.modes[0] = 0;
  for (int i = 0; i < n_operands; ++i) {
    if (!operands[i]) return fail("ib_contract_chain: null operand");
    if (modes[i] < 0 || modes[i] > 3) return fail("ib_contract_chain: operand mode outside 0..3");
    chain.operands[i + 1] = chain.fused.operand[i] = operands[i];
    chain.modes[i + 1] = chain.fused.mode[i] = modes[i];
  }
  chain.fused.n_ops = n_ops;
  for (int j = 0; j < n_ops; ++j) {
    const int op = ops[3 * j], lhs = ops[3 * j + 1], rhs = ops[3 * j + 2];
    if (op != IB_OP_ADD && op != IB_OP_SUB && op != IB_OP_MUL && op != IB_OP_MAX && op != IB_OP_MIN)
      return fail("ib_contract_chain: only + - * > < follow a contraction in its own pass");
    const bool left = lhs == IB_CHAIN_PREV, right = rhs == IB_CHAIN_PREV;
    if (left == right)
      return fail("ib_contract_chain: every operator takes the running value on exactly one side");
    const int other = left ? rhs : lhs;
    if (other != IB_CHAIN_NONE && (other < 0 || other >= n_operands))
      return fail("ib_contract_chain: operand index out of range");
    if (other == IB_CHAIN_NONE && !left)
      return fail("ib_contract_chain: the one-operand form takes the running value");
    chain.fused.op[j] = op;
    chain.fused.which[j] = other == IB_CHAIN_NONE ? -1 : other;
    chain.fused.acc_right[j] = right ? 1 : 0;
    // The same list for ib_map_chain: the stored result is operand 0 and starts the chain.
    auto code = [&](int x) { return x == IB_CHAIN_PREV ? (j == 0 ? 0 : IB_CHAIN_PREV) : x == IB_CHAIN_NONE ? x : x + 1; };
    chain.ops[3 * j] = op;
    chain.ops[3 * j + 1] = code(lhs);
    chain.ops[3 * j + 2] = code(rhs);
  }
  return contract_with_chain(a, b, c, batch, m, n, k, a_kmajor, b_kmajor, precision, col_tile,
                             col_group, &chain, workspace, workspace_bytes, stream);
}

namespace ib {
namespace {

int contract_with_chain(const float* a, const float* b, float* c, size_t batch, size_t m, size_t n,
                        size_t k, int a_kmajor, int b_kmajor, int precision, size_t col_tile,
                        size_t col_group, const ContractChain* chain, void* workspace,
                        size_t workspace_bytes, void* stream) {
  const GemmEpilogue* fused = chain ? &chain->fused : nullptr;
  auto then_chain = [&](int rc) {
    return rc != 0 || !chain ? rc : chain->in_place(c, batch * m, n, stream);
  };
  // The fp32 arm, its k range in parts when the output has too few tiles for the machine and the
  // workspace has room for the copies.
  auto simt = [&](const float* pa, const float* pb, bool a_km, bool b_km, Carver& ws) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t parts = k_parts(batch, m, n, k, 64);
    float* copies = parts > 1 && (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0
                        ? ws.take(batch * parts * m * n)
                        : nullptr;
    if (!copies) return contract_simt(pa, pb, c, batch, m, n, k, a_km, b_km, st);
    if (int rc = contract_simt(pa, pb, copies, batch, m, n, k, a_km, b_km, st, parts)) return rc;
    return sum_partials(copies, c, batch, parts, m * n, st);
  };
  if (col_tile != 0 && col_tile != 128 && col_tile != 256)
    return fail("ib_contract: col_tile must be 0, 128 or 256");
  GemmGeometry geometry;
  geometry.col_tile = static_cast<int>(col_tile);
  geometry.group_n = static_cast<int>(col_group > (1u << 20) ? (1u << 20) : col_group);
  if (batch == 0 || m == 0 || n == 0) return 0;
  if (!a || !b || !c) return fail("ib_contract: null pointer");
  if (too_many_elements({batch, m, k}) || too_many_elements({batch, n, k}) ||
      too_many_elements({batch, m, n}))
    return fail("ib_contract: extents too large (an element count does not fit size_t)");
  if (precision < IB_PRECISION_AUTO || precision > IB_PRECISION_F16)
    return fail("ib_contract: unknown precision");
  if (precision == IB_PRECISION_TF32_F16) precision = IB_PRECISION_TF32;   // attention-only distinction
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (k == 0) {
    cudaError_t err = cudaMemsetAsync(c, 0, batch * m * n * sizeof(float), s);
    return then_chain(err == cudaSuccess ? 0 : fail("ib_contract: memset failed"));
  }
  // Matrix times vector and row-wise dot products have one multiply-add per element read: they
  // are passes over memory, not tile work, and run as a weighted row fold (fp32 throughout,
  // whatever precision was asked for: no arm is less exact), one launch per batch entry when the
  // vector differs between entries.
  {
    const bool dots = m == 1 && n == 1;                       // C[b] = A[b][:] . B[b][:]
    const bool a_rows = !dots && n == 1 && a_kmajor != 0;     // C[b][i] = A[b][i][:] . B[b][:]
    const bool b_rows = !dots && m == 1 && b_kmajor != 0;     // C[b][j] = A[b][:] . B[b][j][:]
    constexpr size_t kMostLaunches = 64;
    if (dots || ((a_rows || b_rows) && batch <= kMostLaunches)) {
      int rc = 0;
      if (dots) {
        const size_t need = long_rows_floats(batch, k);
        float* partials = need && workspace && workspace_bytes / sizeof(float) >= need &&
                                  (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0
                              ? static_cast<float*>(workspace)
                              : nullptr;
        rc = dot_rows(a, b, false, c, batch, k, s, partials);
      } else {
        const size_t rows = a_rows ? m : n;
        for (size_t e = 0; e < batch && rc == 0; ++e)
          rc = dot_rows((a_rows ? a : b) + e * rows * k, (a_rows ? b : a) + e * k, true, c + e * rows,
                        rows, k, s);
      }
      return then_chain(rc);
    }
    // The same with the matrix stored k-major the other way round, [k][rows]: vector times
    // matrix, a weighted fold down the columns.
    const bool a_cols = !dots && n == 1 && a_kmajor == 0;     // C[b][i] = sum_k A[b][k][i] B[b][k]
    const bool b_cols = !dots && m == 1 && b_kmajor == 0;     // C[b][j] = sum_k A[b][k] B[b][k][j]
    if ((a_cols || b_cols) && batch <= kMostLaunches) {
      const size_t cols = a_cols ? m : n;
      const size_t need = dot_leading_axis_floats(k, cols);
      float* partials = workspace && workspace_bytes / sizeof(float) >= need &&
                                (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0
                            ? static_cast<float*>(workspace)
                            : nullptr;
      int rc = 0;
      for (size_t e = 0; e < batch && rc == 0; ++e)
        rc = dot_leading_axis((a_cols ? a : b) + e * k * cols, (a_cols ? b : a) + e * k, c + e * cols, k,
                              cols, partials, s);
      return then_chain(rc);
    }
  }
  const double flop = 2.0 * batch * m * n * k;
  if (precision == IB_PRECISION_AUTO && wants_tensor(precision, flop) && contract_prefers_f16(m, n, k) &&
      workspace && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0 &&
      workspace_bytes >= ib_contract_workspace_bytes(batch, m, n, k, a_kmajor, b_kmajor, IB_PRECISION_F16))
    precision = IB_PRECISION_F16;
  if (precision == IB_PRECISION_F16) {
    // Both operands as fp16 over one power of two per row; the scales return in the epilogue.
    if (reinterpret_cast<uintptr_t>(workspace) & 255u)
      return fail("ib_contract: workspace must be 256-byte aligned");
    Carver ws(workspace, workspace_bytes);
    const char* small = "ib_contract: workspace too small (see ib_contract_workspace_bytes)";
    const size_t kp = round_up(k, 8);
    float* a16 = ws.take((batch * m * kp + 1) / 2);
    float* b16 = ws.take((batch * n * kp + 1) / 2);
    float* a_scale = ws.take(batch * m);
    float* b_scale = ws.take(batch * n);
    if (!a16 || !b16 || !a_scale || !b_scale) return fail(small);
    const float* ak = a;
    const float* bk = b;
    if (!a_kmajor) {
      float* t = ws.take(batch * m * k);
      if (!t) return fail(small);
      if (int rc = transpose_batched(a, t, batch, k, m, k, false, s)) return rc;
      ak = t;
    }
    if (!b_kmajor) {
      float* t = ws.take(batch * n * k);
      if (!t) return fail(small);
      if (int rc = transpose_batched(b, t, batch, k, n, k, false, s)) return rc;
      bk = t;
    }
    if (int rc = convert_f16_rows_scaled(ak, a16, a_scale, batch * m, k, kp, s)) return rc;
    if (int rc = convert_f16_rows_scaled(bk, b16, b_scale, batch * n, k, kp, s)) return rc;
    return gemm_tcgen05_f16(a16, b16, a_scale, b_scale, c, batch, m, n, k, kp, s, geometry, fused);
  }
  if (precision == IB_PRECISION_BF16) {
    if (reinterpret_cast<uintptr_t>(workspace) & 255u)
      return fail("ib_contract: workspace must be 256-byte aligned");
    Carver ws(workspace, workspace_bytes);
    const char* small = "ib_contract: workspace too small (see ib_contract_workspace_bytes)";
    const size_t kp = round_up(k, 8);
    float* a16 = ws.take((batch * m * kp + 1) / 2);
    float* b16 = ws.take((batch * n * kp + 1) / 2);
    if (!a16 || !b16) return fail(small);
    const float* ak = a;
    const float* bk = b;
    if (!a_kmajor) {
      float* t = ws.take(batch * m * k);
      if (!t) return fail(small);
      if (int rc = transpose_batched(a, t, batch, k, m, k, false, s)) return rc;
      ak = t;
    }
    if (!b_kmajor) {
      float* t = ws.take(batch * n * k);
      if (!t) return fail(small);
      if (int rc = transpose_batched(b, t, batch, k, n, k, false, s)) return rc;
      bk = t;
    }
    if (int rc = convert_bf16_rows(ak, a16, batch * m, k, kp, s)) return rc;
    if (int rc = convert_bf16_rows(bk, b16, batch * n, k, kp, s)) return rc;
    return gemm_tcgen05_bf16(a16, b16, c, batch, m, n, k, kp, s, geometry, fused);
  }
  if (wants_tensor(precision, flop) && contract_shape_ok(k)) {
    Carver ws(workspace, workspace_bytes);
    const float* ak = a;
    const float* bk = b;
    if (!a_kmajor) {
      float* t = ws.take(batch * m * k);
      if (!t) return fail("ib_contract: workspace too small (see ib_contract_workspace_bytes)");
      if (int rc = transpose_batched(a, t, batch, k, m, k, false, s)) return rc;   // [k][m] -> [m][k]
      ak = t;
    }
    if (!b_kmajor) {
      float* t = ws.take(batch * n * k);
      if (!t) return fail("ib_contract: workspace too small (see ib_contract_workspace_bytes)");
      if (int rc = transpose_batched(b, t, batch, k, n, k, false, s)) return rc;   // [k][n] -> [n][k]
      bk = t;
    }
    if (gemm_tcgen05_supported(ak, bk, c, m, n, k)) {
      const size_t parts = k_parts_tensor(batch, m, n, k);
      float* copies = parts > 1 ? ws.take(parts * m * n) : nullptr;
      if (!copies) return gemm_tcgen05(ak, bk, c, batch, m, n, k, s, geometry, fused);
      // The parts as batch entries of one launch, then their sum (and the caller's operators
      // on the sum, as a pass of their own).
      // (Should the driver refuse a tensor map whose batch pitch is below its row pitch, the
      // contraction runs whole instead.)
      if (gemm_tcgen05(ak, bk, copies, 1, m, n, k, s, geometry, nullptr, parts) != 0)
        return gemm_tcgen05(ak, bk, c, batch, m, n, k, s, geometry, fused);
      return then_chain(sum_partials(copies, c, 1, parts, m * n, s));
    }
    // Misaligned base pointers: the fp32 arm takes any layout.
    return then_chain(simt(ak, bk, true, true, ws));
  }
  Carver ws(workspace, workspace_bytes);
  return then_chain(simt(a, b, a_kmajor != 0, b_kmajor != 0, ws));
}

}  // namespace
}  // namespace ib

extern "C" size_t ib_attention_workspace_bytes(size_t batch, size_t nq, size_t nk, size_t d,
                                               size_t dv, int v_kmajor, int precision) {
  using namespace ib;
  // Extents whose element counts do not fit size_t: no workspace can serve them (ib_attention
  // refuses the same extents).
  if (too_many_elements({batch, nq, nk}) || too_many_elements({batch, nq, d > dv ? d : dv}) ||
      too_many_elements({batch, nk, d > dv ? d : dv}))
    return SIZE_MAX;
  const double flop = 4.0 * batch * nq * nk * d;
  if (wants_tensor(precision, flop) && attention_shape_ok(d, dv)) {
    // Rounded copy of K, V^T (rounded), and the KV-split partials; bf16 copies
    // are half the size, with pitches rounded up to 8 elements.
    return prepared_kv_bytes(batch, nk, d, dv, attention_arm(precision)) +
           carve_bytes(attention_tcgen05_partial_floats(batch, nq, nk, dv, nullptr));
  }
  // Unfused: S = Q K^T, softmax in place, O = S V.
  size_t bytes = carve_bytes(batch * nq * nk);
  const int sub = wants_tensor(precision, flop) ? IB_PRECISION_TF32 : IB_PRECISION_FP32;
  bytes += ib_contract_workspace_bytes(batch, nq, dv, nk, 1, v_kmajor, sub);
  return bytes;
}

extern "C" int ib_attention_scaled(const float* q, const float* k, const float* v, float* o,
                                   size_t batch, size_t nq, size_t nk, size_t d, size_t dv,
                                   int v_kmajor, int precision, size_t kv_tile,
                                   const float* logit_scale, int logit_divide, void* workspace,
                                   size_t workspace_bytes, void* stream) {
  using namespace ib;
  if (batch == 0 || nq == 0 || dv == 0) return 0;
  if (!q || !k || !v || !o) return fail("ib_attention: null pointer");
  if (nk == 0 || d == 0) return fail("ib_attention: empty key or feature axis");
  if (precision < IB_PRECISION_AUTO || precision > IB_PRECISION_F16)
    return fail("ib_attention: unknown precision");
  if (too_many_elements({batch, nq, nk}) || too_many_elements({batch, nq, d > dv ? d : dv}) ||
      too_many_elements({batch, nk, d > dv ? d : dv}))
    return fail("ib_attention: extents too large (an element count does not fit size_t)");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (reinterpret_cast<uintptr_t>(workspace) & 255u)
    return fail("ib_attention: workspace must be 256-byte aligned");
  Carver ws(workspace, workspace_bytes);
  const double flop = 4.0 * batch * nq * nk * d;
  const bool tensor = wants_tensor(precision, flop);

  if (tensor && attention_shape_ok(d, dv)) {
    PreparedKV kv;
    if (int rc = prepared_kv(k, v, batch, nk, d, dv, v_kmajor != 0, attention_arm(precision), true,
                             ws, &kv, s))
      return rc;
    float* partials = ws.take(attention_tcgen05_partial_floats(batch, nq, nk, dv, nullptr));
    if (!partials)
      return fail("ib_attention: workspace too small (see ib_attention_workspace_bytes)");
    return attention_tcgen05(q, kv.k, kv.vt, o, batch, nq, nk, d, dv, kv.d_pitch, kv.nk_pitch,
                             kv.arm, kv.v_scale, kv.k_tile_scale, logit_scale, logit_divide != 0, true,
                             partials, kv_tile, s);
  }

  float* scores = ws.take(batch * nq * nk);
  if (!scores) return fail("ib_attention: workspace too small (see ib_attention_workspace_bytes)");
  const int sub = tensor ? IB_PRECISION_TF32 : IB_PRECISION_FP32;
  if (int rc = ib_contract(q, k, scores, batch, nq, nk, d, 1, 1, sub, nullptr, 0, stream)) return rc;
  // The scale as the component states it: each logit times (or over) the scalar, in place.
  if (logit_scale)
    if (int rc = ib_map_binary(logit_divide ? IB_OP_DIV : IB_OP_MUL, 1, scores, logit_scale, scores,
                               1, batch * nq * nk, stream))
      return rc;
  if (int rc = ib_row_softmax(scores, scores, batch * nq, nk, stream)) return rc;
  uint8_t* rest = ws.base ? ws.base + ws.used : nullptr;
  return ib_contract(scores, v, o, batch, nq, dv, nk, 1, v_kmajor, sub, rest,
                     workspace_bytes - ws.used, stream);
}

extern "C" int ib_attention(const float* q, const float* k, const float* v, float* o, size_t batch,
                            size_t nq, size_t nk, size_t d, size_t dv, int v_kmajor, int precision,
                            size_t kv_tile, void* workspace, size_t workspace_bytes,
                            void* stream) {
  return ib_attention_scaled(q, k, v, o, batch, nq, nk, d, dv, v_kmajor, precision, kv_tile, nullptr,
                             0, workspace, workspace_bytes, stream);
}

// ---- two-phase form: prepare K and V once, run query blocks against them ----

extern "C" size_t ib_attention_prepare_bytes(size_t batch, size_t nk, size_t d, size_t dv,
                                             int precision) {
  if (ib::too_many_elements({batch, nk, 2 * (d > dv ? d : dv) + 16})) return SIZE_MAX;
  return ib::prepared_kv_bytes(batch, nk, d, dv, ib::attention_arm(precision));
}

extern "C" int ib_attention_prepare(const float* k, const float* v, size_t batch, size_t nk,
                                    size_t d, size_t dv, int v_kmajor, int precision,
                                    void* prepared, size_t prepared_bytes, void* stream) {
  using namespace ib;
  if (batch == 0) return 0;
  if (!k || !v) return fail("ib_attention_prepare: null pointer");
  if (too_many_elements({batch, nk, 2 * (d > dv ? d : dv) + 16}))
    return fail("ib_attention_prepare: extents too large (an element count does not fit size_t)");
  if (nk == 0 || !attention_shape_ok(d, dv))
    return fail("ib_attention_prepare: shape outside the fused kernel's range (d % 4 == 0, d and dv <= 128)");
  if (precision == IB_PRECISION_FP32 || precision < IB_PRECISION_AUTO ||
      precision > IB_PRECISION_F16)
    return fail("ib_attention_prepare: the two-phase form exists for the tensor arms (auto, tf32, bf16, tf32_f16, f16)");
  if (reinterpret_cast<uintptr_t>(prepared) & 255u)
    return fail("ib_attention_prepare: buffer must be 256-byte aligned");
  Carver ws(prepared, prepared_bytes);
  PreparedKV kv;
  return prepared_kv(k, v, batch, nk, d, dv, v_kmajor != 0, attention_arm(precision), true, ws, &kv,
                     static_cast<cudaStream_t>(stream));
}

extern "C" size_t ib_attention_run_workspace_bytes(size_t batch, size_t nq, size_t nk, size_t dv) {
  if (ib::too_many_elements({batch, nq, nk})) return SIZE_MAX;
  return ib::carve_bytes(ib::attention_tcgen05_partial_floats(batch, nq, nk, dv, nullptr));
}

extern "C" int ib_attention_run(const float* q, const void* prepared, float* o, size_t batch,
                                size_t nq, size_t nk, size_t d, size_t dv, int precision,
                                void* workspace, size_t workspace_bytes, void* stream) {
  using namespace ib;
  if (batch == 0 || nq == 0) return 0;
  if (!q || !prepared || !o) return fail("ib_attention_run: null pointer");
  if (too_many_elements({batch, nq, nk}) || too_many_elements({batch, nk, 2 * (d > dv ? d : dv) + 16}))
    return fail("ib_attention_run: extents too large (an element count does not fit size_t)");
  if (nk == 0 || !attention_shape_ok(d, dv))
    return fail("ib_attention_run: shape outside the fused kernel's range (d % 4 == 0, d and dv <= 128)");
  if (precision == IB_PRECISION_FP32 || precision < IB_PRECISION_AUTO ||
      precision > IB_PRECISION_F16)
    return fail("ib_attention_run: the two-phase form exists for the tensor arms (auto, tf32, bf16, tf32_f16, f16)");
  if ((reinterpret_cast<uintptr_t>(prepared) | reinterpret_cast<uintptr_t>(workspace)) & 255u)
    return fail("ib_attention_run: buffers must be 256-byte aligned");
  const AttentionArm arm = attention_arm(precision);
  // Same carving as ib_attention_prepare, without touching the contents.
  Carver held(const_cast<void*>(prepared), prepared_kv_bytes(batch, nk, d, dv, arm));
  PreparedKV kv;
  if (int rc = prepared_kv(nullptr, nullptr, batch, nk, d, dv, false, arm, false, held, &kv, nullptr))
    return rc;
  Carver ws(workspace, workspace_bytes);
  float* partials = ws.take(attention_tcgen05_partial_floats(batch, nq, nk, dv, nullptr));
  if (!partials)
    return fail("ib_attention_run: workspace too small (see ib_attention_run_workspace_bytes)");
  return attention_tcgen05(q, kv.k, kv.vt, o, batch, nq, nk, d, dv, kv.d_pitch, kv.nk_pitch, kv.arm,
                           kv.v_scale, kv.k_tile_scale, nullptr, false, false, partials, 0,
                           static_cast<cudaStream_t>(stream));
}

extern "C" int ib_attention_uses_tensor_arm(size_t batch, size_t nq, size_t nk, size_t d, size_t dv,
                                            int precision) {
  return ib::wants_tensor(precision, 4.0 * batch * nq * nk * d) && ib::attention_shape_ok(d, dv);
}

extern "C" int i_b200_set_reserved_sms(int n) {
  if (n < 0) return ib::fail("i_b200_set_reserved_sms: negative count");
  ib::set_reserved_sms(n);
  return 0;
}

extern "C" int i_b200_reserved_sms(void) { return ib::reserved_sms(); }
