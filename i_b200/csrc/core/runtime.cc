// The C API of include/i.h and include/i_b200.h, and the plan executor.
//
// Mirrors the reference runtime's contract (core/src/lib.rs:61-334): opaque
// component / program handles, combinators that copy their arguments,
// thread-local last error, NULL / -1 / {NULL,0} on failure.  Where the
// reference JIT-compiles C and calls the generated `exec`
// (lib.rs:353-415, 199-225), this runtime walks a Plan and launches the ib_*
// kernels on the current CUDA device.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "i_b200.h"
#include "ir.h"
#include "plan.h"

struct i_component {
  ib::ComponentPtr inner;
};

struct i_program {
  ib::Graph graph;
  ib::Plan plan;
  std::atomic<int> precision{IB_PRECISION_AUTO};
};

namespace ib {

// kernels/device_util.cu: reports a bounded device-side wait that gave up.
int check_device_status(const char* what, cudaStream_t s);

namespace {
thread_local std::string g_error;
thread_local bool g_has_error = false;
std::atomic<size_t> g_launches{0};
}  // namespace

void set_error(const std::string& message) {
  g_error = message;
  g_error.erase(std::remove(g_error.begin(), g_error.end(), '\0'), g_error.end());
  g_has_error = true;
}

void count_launch(size_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

namespace {

using Shape = std::vector<size_t>;

size_t product(const Shape& s, size_t from = 0, size_t to = static_cast<size_t>(-1)) {
  size_t p = 1;
  for (size_t i = from; i < s.size() && i < to; ++i) p *= s[i];
  return p;
}

int op_code(Op op) {
  switch (op) {
    case Op::Add: return IB_OP_ADD;
    case Op::Mul: return IB_OP_MUL;
    case Op::Sub: return IB_OP_SUB;
    case Op::Div: return IB_OP_DIV;
    case Op::Max: return IB_OP_MAX;
    case Op::Min: return IB_OP_MIN;
    case Op::Pow: return IB_OP_POW;
    case Op::Log: return IB_OP_LOG;
    case Op::Gt: return IB_OP_GT;
    case Op::Ge: return IB_OP_GE;
    case Op::Lt: return IB_OP_LT;
    case Op::Le: return IB_OP_LE;
    case Op::Eq: return IB_OP_EQ;
    case Op::Ne: return IB_OP_NE;
    case Op::And: return IB_OP_AND;
    case Op::Or: return IB_OP_OR;
    case Op::Xor: return IB_OP_XOR;
    default: return IB_OP_NOT;
  }
}

int default_precision() {
  const char* env = std::getenv("I_B200_PRECISION");
  if (!env) return IB_PRECISION_AUTO;
  std::string v(env);
  if (v == "fp32") return IB_PRECISION_FP32;
  if (v == "tf32") return IB_PRECISION_TF32;
  if (v == "bf16") return IB_PRECISION_BF16;
  if (v == "tf32_f16") return IB_PRECISION_TF32_F16;
  if (v == "f16") return IB_PRECISION_F16;
  return IB_PRECISION_AUTO;
}

// Shapes of every buffer a plan touches, derived from the input shapes.
struct ShapeTable {
  std::vector<Shape> inputs;
  std::vector<Shape> nodes;
  std::vector<bool> node_known;

  const Shape* get(const Source& s) const {
    if (s.is_input) return s.index < inputs.size() ? &inputs[s.index] : nullptr;
    return (s.index < nodes.size() && node_known[s.index]) ? &nodes[s.index] : nullptr;
  }
};

// Extents of a step's local indexes, first operand mentioning an index wins
// (reference: compiler/src/lower/node_to_stage.rs:232-261); later mentions
// must agree.
bool step_extents(const Step& step, const ShapeTable& shapes, std::vector<size_t>* extent,
                  std::string* err) {
  extent->assign(step.rank, 0);
  std::vector<bool> known(step.rank, false);
  for (size_t a = 0; a < step.in.size(); ++a) {
    const Access& acc = step.in[a];
    const Shape* shape = shapes.get(acc.buffer);
    if (!shape) {
      *err = "internal: operand shape unknown";
      return false;
    }
    if (shape->size() != acc.index.size()) {
      *err = "operand " + std::to_string(a) + " has rank " + std::to_string(shape->size()) +
             " but its pattern has " + std::to_string(acc.index.size()) + " axes";
      return false;
    }
    for (size_t p = 0; p < acc.index.size(); ++p) {
      size_t x = acc.index[p];
      if (x >= step.rank) continue;  // attention keeps V in its own index space
      if (!known[x]) {
        (*extent)[x] = (*shape)[p];
        known[x] = true;
      } else if ((*extent)[x] != (*shape)[p]) {
        *err = "axis extent mismatch: " + std::to_string((*extent)[x]) + " vs " +
               std::to_string((*shape)[p]);
        return false;
      }
    }
  }
  return true;
}

struct AttentionDims {
  size_t batch, nq, nk, d, dv;
  bool v_kmajor;
};

bool attention_dims(const Step& step, const ShapeTable& shapes, AttentionDims* out, Shape* oshape,
                    std::string* err) {
  const Shape* q = shapes.get(step.in[0].buffer);
  const Shape* k = shapes.get(step.in[1].buffer);
  const Shape* v = shapes.get(step.in[2].buffer);
  const size_t nb = step.form.n_batch;
  if (!q || !k || !v || q->size() != nb + 2 || k->size() != nb + 2 || v->size() != nb + 2) {
    *err = "attention operands must have rank " + std::to_string(nb + 2);
    return false;
  }
  for (size_t i = 0; i < nb; ++i)
    if ((*q)[i] != (*k)[i] || (*q)[i] != (*v)[i]) {
      *err = "attention batch axes differ between operands";
      return false;
    }
  if (step.in.size() == 4) {
    const Shape* c = shapes.get(step.in[3].buffer);
    if (!c || !c->empty()) {
      *err = "the scale on the attention logits must be a scalar";
      return false;
    }
  }
  out->batch = product(*q, 0, nb);
  out->nq = (*q)[nb];
  out->d = (*q)[nb + 1];
  out->nk = (*k)[nb];
  out->v_kmajor = step.form2.b_kmajor;
  const size_t v_keys = out->v_kmajor ? (*v)[nb + 1] : (*v)[nb];
  out->dv = out->v_kmajor ? (*v)[nb] : (*v)[nb + 1];
  if ((*k)[nb + 1] != out->d || v_keys != out->nk) {
    *err = "attention operand extents do not agree";
    return false;
  }
  oshape->assign(q->begin(), q->begin() + nb);
  oshape->push_back(out->nq);
  oshape->push_back(out->dv);
  return true;
}

bool infer_shapes(const Plan& plan, const i_tensor* inputs, size_t input_count, ShapeTable* table,
                  std::string* err) {
  if (input_count != plan.n_inputs) {
    *err = "expected " + std::to_string(plan.n_inputs) + " inputs, got " +
           std::to_string(input_count);
    return false;
  }
  table->inputs.resize(plan.n_inputs);
  for (size_t i = 0; i < plan.n_inputs; ++i) {
    if (inputs[i].rank > 0 && !inputs[i].shape) {
      *err = "input " + std::to_string(i) + " has a null shape";
      return false;
    }
    table->inputs[i].assign(inputs[i].shape, inputs[i].shape + inputs[i].rank);
  }
  table->nodes.assign(plan.n_nodes, Shape());
  table->node_known.assign(plan.n_nodes, false);
  for (const Step& step : plan.steps) {
    Shape out;
    if (step.kind == StepKind::Attention) {
      AttentionDims dims;
      if (!attention_dims(step, *table, &dims, &out, err)) return false;
    } else {
      std::vector<size_t> extent;
      if (!step_extents(step, *table, &extent, err)) return false;
      for (size_t x : step.out.index) out.push_back(extent[x]);
      // Operands of a contraction's epilogue are indexed over the result's axes.
      for (const Access& acc : step.epilogue_in) {
        const Shape* shape = table->get(acc.buffer);
        if (!shape) {
          *err = "internal: operand shape unknown";
          return false;
        }
        if (shape->size() != acc.index.size()) {
          *err = "operand has rank " + std::to_string(shape->size()) + " but its pattern has " +
                 std::to_string(acc.index.size()) + " axes";
          return false;
        }
        for (size_t p = 0; p < acc.index.size(); ++p)
          if (acc.index[p] >= out.size() || (*shape)[p] != out[acc.index[p]]) {
            *err = "axis extent mismatch: " +
                   std::to_string(acc.index[p] < out.size() ? out[acc.index[p]] : 0) + " vs " +
                   std::to_string((*shape)[p]);
            return false;
          }
      }
    }
    table->nodes[step.out.buffer.index] = out;
    table->node_known[step.out.buffer.index] = true;
  }
  return true;
}

// ---- execution ------------------------------------------------------------

// Scratch and staging buffers come from a per-device memory pool owned by this
// library.  Its release threshold is unlimited, so memory freed at the end of
// one call is reused by the next instead of going back to the driver at every
// stream synchronisation (the default pool does that, at milliseconds a call).
cudaMemPool_t library_pool() {
  static std::mutex mutex;
  static std::map<int, cudaMemPool_t> pools;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(mutex);
  auto it = pools.find(dev);
  if (it != pools.end()) return it->second;
  cudaMemPoolProps props = {};
  props.allocType = cudaMemAllocationTypePinned;
  props.handleTypes = cudaMemHandleTypeNone;
  props.location.type = cudaMemLocationTypeDevice;
  props.location.id = dev;
  cudaMemPool_t pool = nullptr;
  if (cudaMemPoolCreate(&pool, &props) != cudaSuccess) {
    cudaGetLastError();
    pool = nullptr;
  } else {
    unsigned long long keep = ~0ull;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
  }
  pools[dev] = pool;
  return pool;
}

struct DeviceBuffers {
  std::vector<const float*> inputs;
  std::vector<float*> nodes;
  std::vector<void*> owned;     // freed (stream-ordered) after the run
  cudaStream_t stream = nullptr;

  const float* get(const Source& s) const { return s.is_input ? inputs[s.index] : nodes[s.index]; }

  float* alloc(size_t bytes, std::string* err) {
    void* p = nullptr;
    if (bytes == 0) bytes = 4;
    cudaMemPool_t pool = library_pool();
    cudaError_t rc = pool ? cudaMallocFromPoolAsync(&p, bytes, pool, stream)
                          : cudaMallocAsync(&p, bytes, stream);
    if (rc != cudaSuccess) {
      *err = std::string("device allocation of ") + std::to_string(bytes) +
             " bytes failed: " + cudaGetErrorString(rc);
      cudaGetLastError();
      return nullptr;
    }
    owned.push_back(p);
    return static_cast<float*>(p);
  }

  void release() {
    for (void* p : owned) cudaFreeAsync(p, stream);
    owned.clear();
  }
};

std::vector<ptrdiff_t> dense_strides(const Shape& s) {
  std::vector<ptrdiff_t> st(s.size(), 1);
  for (size_t i = s.size(); i-- > 1;) st[i - 1] = st[i] * static_cast<ptrdiff_t>(s[i]);
  return st;
}

// Stride of step index x inside an operand (sum over repeated mentions).
ptrdiff_t stride_of(const Access& acc, const Shape& shape, size_t x) {
  std::vector<ptrdiff_t> st = dense_strides(shape);
  ptrdiff_t total = 0;
  for (size_t p = 0; p < acc.index.size(); ++p)
    if (acc.index[p] == x) total += st[p];
  return total;
}

bool is_prefix(const std::vector<size_t>& small, const std::vector<size_t>& big) {
  if (small.size() >= big.size()) return false;
  return std::equal(small.begin(), small.end(), big.begin());
}

bool is_suffix(const std::vector<size_t>& small, const std::vector<size_t>& big) {
  if (small.size() >= big.size() || small.empty()) return false;
  return std::equal(small.rbegin(), small.rend(), big.rbegin());
}

int run_map(const Step& step, const ShapeTable& shapes, const std::vector<size_t>& extent,
            DeviceBuffers& dev, float* out, const Shape& oshape) {
  const int op = op_code(step.op);
  const size_t n = product(oshape);
  const Access& a = step.in[0];
  const float* pa = dev.get(a.buffer);
  void* stream = dev.stream;
  (void)extent;
  if (step.in.size() == 1) {
    if (a.index == step.out.index) return ib_map_unary(op, pa, out, n, stream);
    // A copy with the last two axes exchanged (`ij~ji`, `bij~bji`): the tiled transpose.
    const size_t r = step.out.index.size();
    if ((step.op == Op::Add || step.op == Op::Mul) && r >= 2 && a.index.size() == r &&
        std::equal(a.index.begin(), a.index.end() - 2, step.out.index.begin()) &&
        a.index[r - 2] == step.out.index[r - 1] && a.index[r - 1] == step.out.index[r - 2] &&
        a.index[r - 2] != a.index[r - 1] && (oshape[r - 1] + 63) / 64 <= 65535) {   // the tile kernel's grid
      const size_t out_rows = oshape[r - 2], out_cols = oshape[r - 1];
      return ib_transpose(pa, out, n / (out_rows * out_cols ? out_rows * out_cols : 1), out_cols, out_rows,
                          stream);
    }
  } else {
    const Access& b = step.in[1];
    const float* pb = dev.get(b.buffer);
    const auto& full = step.out.index;
    const bool a_full = a.index == full, b_full = b.index == full;
    if (a_full && b_full) return ib_map_binary(op, 0, pa, pb, out, 1, n, stream);
    if (a_full && is_prefix(b.index, full)) {
      size_t rows = product(oshape, 0, b.index.size());
      return ib_map_binary(op, 1, pa, pb, out, rows, n / (rows ? rows : 1), stream);
    }
    if (b_full && is_prefix(a.index, full)) {
      size_t rows = product(oshape, 0, a.index.size());
      return ib_map_binary(op, 2, pa, pb, out, rows, n / (rows ? rows : 1), stream);
    }
    if (a_full && is_suffix(b.index, full)) {
      size_t cols = product(oshape, full.size() - b.index.size());
      return ib_map_binary(op, 3, pa, pb, out, n / (cols ? cols : 1), cols, stream);
    }
    if (b_full && is_suffix(a.index, full)) {
      size_t cols = product(oshape, full.size() - a.index.size());
      return ib_map_binary(op, 4, pa, pb, out, n / (cols ? cols : 1), cols, stream);
    }
  }
  // General case: strides per result dimension.
  if (oshape.size() > IB_MAX_RANK) {
    set_error("maps of more than 8 axes are not supported");
    return -1;
  }
  std::vector<ptrdiff_t> sa(oshape.size()), sb(oshape.size());
  const Shape& shape_a = *shapes.get(a.buffer);
  for (size_t p = 0; p < oshape.size(); ++p) sa[p] = stride_of(a, shape_a, step.out.index[p]);
  const float* pb = nullptr;
  if (step.in.size() == 2) {
    const Access& b = step.in[1];
    pb = dev.get(b.buffer);
    const Shape& shape_b = *shapes.get(b.buffer);
    for (size_t p = 0; p < oshape.size(); ++p) sb[p] = stride_of(b, shape_b, step.out.index[p]);
  }
  return ib_map_strided(op, pa, pb, out, static_cast<int>(oshape.size()), oshape.data(), sa.data(),
                        pb ? sb.data() : nullptr, stream);
}

// How a chain kernel addresses an operand of a `rank`-axis index space: 0 the full tensor,
// 1 one value per row (every axis but the last), 2 one value per column (the last axis),
// 3 a scalar.  The planner admits only these forms.
int chain_operand_mode(const Access& acc, size_t rank) {
  if (acc.index.size() == rank) return 0;
  if (rank >= 2 && acc.index.size() == 1 && acc.index[0] == rank - 1) return 2;
  return acc.index.empty() ? 3 : 1;
}

// MapChain: `oshape` is the result's shape.  ChainReduce: the result is one value per row and the
// column count comes from an operand that carries the folded (last) axis.
int run_map_chain(const Step& step, const ShapeTable& shapes, DeviceBuffers& dev, float* out,
                  const Shape& oshape) {
  size_t rows, cols;
  if (step.kind == StepKind::ChainReduce) {
    rows = product(oshape);
    cols = 1;
    for (const Access& acc : step.in)
      if (!acc.index.empty() && acc.index.back() == step.rank - 1)
        cols = shapes.get(acc.buffer)->back();
  } else {
    cols = oshape.empty() ? 1 : oshape.back();
    rows = cols ? product(oshape) / cols : 0;
  }
  std::vector<const float*> operands;
  std::vector<int> modes;
  for (const Access& acc : step.in) {
    operands.push_back(dev.get(acc.buffer));
    modes.push_back(chain_operand_mode(acc, step.rank));
  }
  std::vector<int> ops;
  for (const ChainOp& c : step.chain) {
    ops.push_back(op_code(c.op));
    ops.push_back(c.lhs == kChainPrev ? IB_CHAIN_PREV : c.lhs);
    ops.push_back(c.rhs == kChainPrev ? IB_CHAIN_PREV : c.rhs == kChainNone ? IB_CHAIN_NONE : c.rhs);
  }
  if (step.kind == StepKind::ChainReduce)
    return ib_reduce_rows_chain(op_code(step.op), static_cast<int>(step.chain.size()), ops.data(),
                                static_cast<int>(operands.size()), operands.data(), modes.data(),
                                out, rows, cols, dev.stream);
  return ib_map_chain(static_cast<int>(step.chain.size()), ops.data(),
                      static_cast<int>(operands.size()), operands.data(), modes.data(), out, rows,
                      cols, dev.stream);
}

int run_reduce(const Step& step, const ShapeTable& shapes, const std::vector<size_t>& extent,
               DeviceBuffers& dev, float* out, const Shape& oshape) {
  const int op = op_code(step.op);
  const Access& a = step.in[0];
  const float* pa = dev.get(a.buffer);
  const Shape& shape_a = *shapes.get(a.buffer);
  const size_t kept = step.out.index.size();
  // Fast path: the kept axes lead the operand in output order; the rest fold.
  if (a.index.size() == step.rank && kept <= a.index.size() &&
      std::equal(step.out.index.begin(), step.out.index.end(), a.index.begin())) {
    size_t rows = product(oshape);
    size_t cols = product(shape_a, kept);
    const size_t ws_bytes = ib_reduce_rows_workspace_bytes(rows, cols);
    if (ws_bytes == 0) return ib_reduce_rows(op, pa, out, rows, cols, dev.stream);
    std::string err;
    void* ws = dev.alloc(ws_bytes, &err);
    if (!ws) {
      set_error(err);
      return -1;
    }
    return ib_reduce_rows_split(op, pa, out, rows, cols, ws, ws_bytes, dev.stream);
  }
  // The folded axes stand together in the operand with kept axes behind them, and the kept axes
  // keep their order (`+ij~j`, `+bij~ij`, `+bij~bj`): a fold down the columns of [kept in front]
  // arrays of shape [folded][kept behind].
  if (a.index.size() == step.rank && kept >= 1 && kept < a.index.size() &&
      std::set<size_t>(a.index.begin(), a.index.end()).size() == a.index.size()) {
    size_t front = 0;
    while (front < kept && a.index[front] == step.out.index[front]) ++front;
    const size_t folded = a.index.size() - kept;
    const size_t behind = kept - front;
    if (behind >= 1 && product(shape_a, 0, front) <= 65535 &&        // arrays are a grid axis of the kernel
        std::equal(step.out.index.begin() + front, step.out.index.end(), a.index.begin() + front + folded)) {
      const size_t batch = product(shape_a, 0, front);
      const size_t rows = product(shape_a, front, front + folded);
      const size_t cols = product(shape_a, front + folded);
      const size_t ws_bytes = ib_reduce_leading_workspace_bytes(batch, rows, cols);
      std::string err;
      void* ws = nullptr;
      if (ws_bytes && ws_bytes != SIZE_MAX && !(ws = dev.alloc(ws_bytes, &err))) {
        set_error(err);
        return -1;
      }
      return ib_reduce_leading(op, pa, out, batch, rows, cols, ws, ws ? ws_bytes : 0, dev.stream);
    }
  }
  std::vector<size_t> red_idx;
  for (size_t x = 0; x < step.rank; ++x)
    if (std::find(step.out.index.begin(), step.out.index.end(), x) == step.out.index.end())
      red_idx.push_back(x);
  if (kept > IB_MAX_RANK || red_idx.size() > IB_MAX_RANK) {
    set_error("reductions over more than 8 axes are not supported");
    return -1;
  }
  std::vector<ptrdiff_t> ks(kept), rs(red_idx.size());
  std::vector<size_t> re(red_idx.size());
  for (size_t p = 0; p < kept; ++p) ks[p] = stride_of(a, shape_a, step.out.index[p]);
  for (size_t p = 0; p < red_idx.size(); ++p) {
    rs[p] = stride_of(a, shape_a, red_idx[p]);
    re[p] = extent[red_idx[p]];
  }
  return ib_reduce_strided(op, pa, out, static_cast<int>(kept), oshape.data(), ks.data(),
                           static_cast<int>(red_idx.size()), re.data(), rs.data(), dev.stream);
}

int run_contract(const Step& step, const std::vector<size_t>& extent, DeviceBuffers& dev,
                 float* out, int precision, std::string* err) {
  const ContractForm& f = step.form;
  size_t batch = 1;
  for (size_t i = 0; i < f.n_batch; ++i) batch *= extent[step.in[0].index[i]];
  size_t m = f.has_m ? extent[f.m] : 1;
  size_t n = f.has_n ? extent[f.n] : 1;
  const size_t k = extent[f.k];
  const float* a = dev.get(step.in[0].buffer);
  const float* b = dev.get(step.in[1].buffer);
  bool a_kmajor = f.a_kmajor, b_kmajor = f.b_kmajor;
  if (f.swap_out) {  // result stored [n][m]: compute B A^T instead
    std::swap(a, b);
    std::swap(m, n);
    std::swap(a_kmajor, b_kmajor);
  }
  const size_t ws_bytes = ib_contract_workspace_bytes(batch, m, n, k, a_kmajor, b_kmajor, precision);
  void* ws = nullptr;
  if (ws_bytes && !(ws = dev.alloc(ws_bytes, err))) {
    set_error(*err);
    return -1;
  }
  // A result stored [n][m] swaps the roles of the two output axes, and with them what the
  // schedule said about rows and columns; the geometry is then left to the kernel.
  const Geometry g = f.swap_out ? Geometry{} : choose_geometry(StepKind::Contract, step.hint);
  if (step.chain.empty())
    return ib_contract_tiled(a, b, out, batch, m, n, k, a_kmajor, b_kmajor, precision, g.col_tile,
                             g.col_group, ws, ws_bytes, dev.stream);
  // Pointwise operators on the result (the planner only attaches them to a result stored
  // [.., m, n]); their operands are addressed against the result's rows and columns.
  std::vector<const float*> operands;
  std::vector<int> modes;
  for (const Access& acc : step.epilogue_in) {
    operands.push_back(dev.get(acc.buffer));
    modes.push_back(chain_operand_mode(acc, step.chain_rank));
  }
  std::vector<int> ops;
  for (const ChainOp& c : step.chain) {
    ops.push_back(op_code(c.op));
    ops.push_back(c.lhs == kChainPrev ? IB_CHAIN_PREV : c.lhs);
    ops.push_back(c.rhs == kChainPrev ? IB_CHAIN_PREV : c.rhs == kChainNone ? IB_CHAIN_NONE : c.rhs);
  }
  return ib_contract_chain(a, b, out, batch, m, n, k, a_kmajor, b_kmajor, precision, g.col_tile,
                           g.col_group, static_cast<int>(step.chain.size()), ops.data(),
                           static_cast<int>(operands.size()), operands.data(), modes.data(), ws,
                           ws_bytes, dev.stream);
}

int run_attention(const Step& step, const ShapeTable& shapes, DeviceBuffers& dev, float* out,
                  int precision, std::string* err) {
  AttentionDims dims;
  Shape oshape;
  if (!attention_dims(step, shapes, &dims, &oshape, err)) {
    set_error(*err);
    return -1;
  }
  const size_t ws_bytes = ib_attention_workspace_bytes(dims.batch, dims.nq, dims.nk, dims.d, dims.dv,
                                                      dims.v_kmajor, precision);
  void* ws = nullptr;
  if (ws_bytes && !(ws = dev.alloc(ws_bytes, err))) {
    set_error(*err);
    return -1;
  }
  const float* scale = step.in.size() == 4 ? dev.get(step.in[3].buffer) : nullptr;
  return ib_attention_scaled(dev.get(step.in[0].buffer), dev.get(step.in[1].buffer),
                             dev.get(step.in[2].buffer), out, dims.batch, dims.nq, dims.nk, dims.d,
                             dims.dv, dims.v_kmajor, precision,
                             choose_geometry(StepKind::Attention, step.hint).kv_granule, scale,
                             step.op == Op::Div, ws, ws_bytes, dev.stream);
}

// Runs the plan on device pointers.  `outputs[i]` receives graph output i.
int run_plan(const i_program* program, const ShapeTable& shapes, const float* const* inputs,
             float* const* outputs, cudaStream_t stream) {
  const Plan& plan = program->plan;
  const int precision = program->precision.load();
  DeviceBuffers dev;
  dev.stream = stream;
  dev.inputs.assign(inputs, inputs + plan.n_inputs);
  dev.nodes.assign(plan.n_nodes, nullptr);
  // A node that is a graph output is written straight into the first output
  // slot that names it.
  std::map<size_t, float*> direct;
  for (size_t o = 0; o < plan.outputs.size(); ++o)
    if (!plan.outputs[o].is_input && !direct.count(plan.outputs[o].index))
      direct[plan.outputs[o].index] = outputs[o];

  std::string err;
  int rc = 0;
  for (const Step& step : plan.steps) {
    const size_t node = step.out.buffer.index;
    const Shape& oshape = shapes.nodes[node];
    float* out = nullptr;
    auto it = direct.find(node);
    if (it != direct.end()) {
      out = it->second;
    } else if (!(out = dev.alloc(product(oshape) * sizeof(float), &err))) {
      set_error(err);
      rc = -1;
      break;
    }
    dev.nodes[node] = out;
    if (product(oshape) == 0) continue;
    std::vector<size_t> extent;
    if (step.kind != StepKind::Attention && !step_extents(step, shapes, &extent, &err)) {
      set_error(err);
      rc = -1;
      break;
    }
    switch (step.kind) {
      case StepKind::Map: rc = run_map(step, shapes, extent, dev, out, oshape); break;
      case StepKind::MapChain:
      case StepKind::ChainReduce: rc = run_map_chain(step, shapes, dev, out, oshape); break;
      case StepKind::Reduce: rc = run_reduce(step, shapes, extent, dev, out, oshape); break;
      case StepKind::Contract: rc = run_contract(step, extent, dev, out, precision, &err); break;
      case StepKind::RowSoftmax: {
        const Shape& xs = *shapes.get(step.in[0].buffer);
        size_t cols = xs.empty() ? 1 : xs.back();
        rc = ib_row_softmax(dev.get(step.in[0].buffer), out, cols ? product(xs) / cols : 0, cols,
                            stream);
        break;
      }
      case StepKind::Attention: rc = run_attention(step, shapes, dev, out, precision, &err); break;
    }
    if (rc) break;
  }
  // Outputs that are graph inputs, or repeat an earlier output, are copies.
  for (size_t o = 0; rc == 0 && o < plan.outputs.size(); ++o) {
    const Source& src = plan.outputs[o];
    const float* from = src.is_input ? dev.inputs[src.index] : dev.nodes[src.index];
    if (from == outputs[o]) continue;
    const Shape& shape = src.is_input ? shapes.inputs[src.index] : shapes.nodes[src.index];
    size_t bytes = product(shape) * sizeof(float);
    if (bytes && cudaMemcpyAsync(outputs[o], from, bytes, cudaMemcpyDeviceToDevice, stream) !=
                     cudaSuccess) {
      set_error("copying an output failed");
      rc = -1;
    }
  }
  dev.release();
  return rc;
}

bool device_available(std::string* why) {
  int count = 0;
  cudaError_t rc = cudaGetDeviceCount(&count);
  if (rc != cudaSuccess || count == 0) {
    *why = std::string("no usable CUDA device (") +
           (rc != cudaSuccess ? cudaGetErrorString(rc) : "device count is 0") +
           "); this runtime has no CPU path";
    cudaGetLastError();
    return false;
  }
  return true;
}

bool is_device_pointer(const void* p) {
  if (!p) return false;
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

cudaStream_t thread_stream() {
  thread_local std::map<int, cudaStream_t> streams;
  int dev = 0;
  cudaGetDevice(&dev);
  auto it = streams.find(dev);
  if (it != streams.end()) return it->second;
  cudaStream_t s = nullptr;
  if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) s = nullptr;
  streams[dev] = s;
  return s;
}

// ---- host operands: copies overlapped with the kernels -----------------------
//
// A program that is one fused attention step, called with host buffers, spends
// more time on the PCIe copies than in the kernel.  Query rows are independent
// and so are heads (ilang-python/annotated-flashattn.c:92-127, 240-307), so the
// call is cut into blocks and run as a three-stage pipeline on three streams:
// upload block c+1 | attend block c | download block c-1.
//   one head:  K and V go up first and are prepared once; blocks are ranges of
//              query rows (ib_attention_prepare / ib_attention_run);
//   many heads: blocks are ranges of heads, each a complete ib_attention.
struct SideStreams {
  cudaStream_t in = nullptr, out = nullptr;
  std::vector<cudaEvent_t> events;
  size_t used = 0;
  cudaEvent_t event() {
    if (used == events.size()) {
      cudaEvent_t e = nullptr;
      if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return nullptr;
      events.push_back(e);
    }
    return events[used++];
  }
};

SideStreams* side_streams() {
  thread_local std::map<int, SideStreams> per_device;
  int dev = 0;
  cudaGetDevice(&dev);
  SideStreams& s = per_device[dev];
  if (!s.in && cudaStreamCreateWithFlags(&s.in, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
  if (!s.out && cudaStreamCreateWithFlags(&s.out, cudaStreamNonBlocking) != cudaSuccess)
    return nullptr;
  s.used = 0;
  return &s;
}

size_t host_pipeline_blocks() {
  static const size_t blocks = [] {
    const char* v = std::getenv("I_B200_HOST_BLOCKS");     // 1 switches the pipeline off
    long n = v ? std::atol(v) : 4;
    return static_cast<size_t>(n < 1 ? 1 : (n > 64 ? 64 : n));
  }();
  return blocks;
}

constexpr size_t kPipelineMinBytes = 4u << 20;   // below this the copies are too short to split

// Returns 1 when the call is not of this form (the caller takes the plain path),
// 0 on success, -1 on error.  All pointers are host memory.
int pipelined_host_attention(const i_program* program, const ShapeTable& shapes,
                             const i_tensor* inputs, size_t input_count, i_tensor_mut* outputs,
                             size_t output_count, cudaStream_t stream) {
  const Plan& plan = program->plan;
  if (plan.steps.size() != 1 || plan.steps[0].kind != StepKind::Attention) return 1;
  if (output_count != 1 || plan.outputs.size() != 1 || plan.outputs[0].is_input) return 1;
  const Step& step = plan.steps[0];
  if (step.in.size() != 3) return 1;                   // scaled logits: the plain path
  if (plan.outputs[0].index != step.out.buffer.index) return 1;
  for (int a = 0; a < 3; ++a)
    if (!step.in[a].buffer.is_input || step.in[a].buffer.index >= input_count) return 1;
  const size_t iq = step.in[0].buffer.index, ik = step.in[1].buffer.index,
               iv = step.in[2].buffer.index;
  if (iq == ik || iq == iv || ik == iv) return 1;
  AttentionDims dims;
  Shape oshape;
  std::string err;
  if (!attention_dims(step, shapes, &dims, &oshape, &err)) return 1;   // reported by the plain path
  const int precision = program->precision.load();
  if (!ib_attention_uses_tensor_arm(dims.batch, dims.nq, dims.nk, dims.d, dims.dv, precision)) return 1;
  const size_t q_floats = dims.nq * dims.d, k_floats = dims.nk * dims.d, v_floats = dims.nk * dims.dv,
               o_floats = dims.nq * dims.dv;                           // per head
  if (dims.batch * (q_floats + k_floats + v_floats + o_floats) * sizeof(float) < kPipelineMinBytes)
    return 1;
  size_t blocks = host_pipeline_blocks();
  const bool by_rows = dims.batch == 1;
  size_t rows_per_block = 0, heads_per_block = 0;
  if (by_rows) {
    const size_t tiles = (dims.nq + 127) / 128;
    blocks = std::min(blocks, tiles / 8);                  // at least 1024 rows a block
    if (blocks < 2) return 1;
    rows_per_block = (tiles + blocks - 1) / blocks * 128;
    blocks = (dims.nq + rows_per_block - 1) / rows_per_block;
  } else {
    blocks = std::min(blocks * 2, dims.batch);
    if (blocks < 2) return 1;
    heads_per_block = (dims.batch + blocks - 1) / blocks;
    blocks = (dims.batch + heads_per_block - 1) / heads_per_block;
  }
  for (size_t i : {iq, ik, iv})
    if (!inputs[i].data) {
      set_error("input " + std::to_string(i) + " has null data");
      return -1;
    }
  if (!outputs[0].data) {
    set_error("output 0 has null data");
    return -1;
  }
  SideStreams* side = side_streams();
  if (!side) return 1;

  const float* hq = inputs[iq].data;
  const float* hk = inputs[ik].data;
  const float* hv = inputs[iv].data;
  float* ho = outputs[0].data;
  DeviceBuffers dev;
  dev.stream = stream;
  float* dq = dev.alloc(dims.batch * q_floats * sizeof(float), &err);
  float* dk = dev.alloc(dims.batch * k_floats * sizeof(float), &err);
  float* dv = dev.alloc(dims.batch * v_floats * sizeof(float), &err);
  float* dout = dev.alloc(dims.batch * o_floats * sizeof(float), &err);
  const size_t block_heads = by_rows ? 1 : heads_per_block;
  const size_t block_rows = by_rows ? rows_per_block : dims.nq;
  const size_t prep_bytes =
      by_rows ? ib_attention_prepare_bytes(1, dims.nk, dims.d, dims.dv, precision) : 0;
  const size_t ws_bytes =
      by_rows ? ib_attention_run_workspace_bytes(1, block_rows, dims.nk, dims.dv)
              : ib_attention_workspace_bytes(block_heads, dims.nq, dims.nk, dims.d, dims.dv,
                                             dims.v_kmajor, precision);
  float* prepared = by_rows ? dev.alloc(prep_bytes, &err) : nullptr;
  float* ws = dev.alloc(ws_bytes, &err);
  int rc = 0;
  if (!dq || !dk || !dv || !dout || !ws || (by_rows && !prepared)) {
    set_error(err);
    rc = -1;
  }
  auto ok = [&](cudaError_t e, const char* what) {
    if (e == cudaSuccess || rc) return;
    set_error(std::string(what) + ": " + cudaGetErrorString(e));
    rc = -1;
  };
  auto signal = [&](cudaStream_t from, cudaStream_t to, const char* what) {
    cudaEvent_t e = side->event();
    if (!e) {
      ok(cudaErrorMemoryAllocation, what);
      return;
    }
    ok(cudaEventRecord(e, from), what);
    ok(cudaStreamWaitEvent(to, e, 0), what);
  };
  const size_t f = sizeof(float);
  if (rc == 0) {
    // The buffers were allocated in `stream` order; the copy streams start after that point.
    signal(stream, side->in, "ordering the upload stream");
    signal(stream, side->out, "ordering the download stream");
    if (by_rows) {
      ok(cudaMemcpyAsync(dk, hk, k_floats * f, cudaMemcpyHostToDevice, side->in), "uploading K");
      ok(cudaMemcpyAsync(dv, hv, v_floats * f, cudaMemcpyHostToDevice, side->in), "uploading V");
      signal(side->in, stream, "ordering the preparation");
      if (rc == 0)
        rc = ib_attention_prepare(dk, dv, 1, dims.nk, dims.d, dims.dv, dims.v_kmajor, precision,
                                  prepared, prep_bytes, stream);
    }
    for (size_t c = 0; rc == 0 && c < blocks; ++c) {
      if (by_rows) {
        const size_t r0 = c * block_rows, rows = std::min(block_rows, dims.nq - r0);
        ok(cudaMemcpyAsync(dq + r0 * dims.d, hq + r0 * dims.d, rows * dims.d * f,
                           cudaMemcpyHostToDevice, side->in), "uploading Q");
        signal(side->in, stream, "ordering a query block");
        if (rc == 0)
          rc = ib_attention_run(dq + r0 * dims.d, prepared, dout + r0 * dims.dv, 1, rows, dims.nk,
                                dims.d, dims.dv, precision, ws, ws_bytes, stream);
        signal(stream, side->out, "ordering a download");
        ok(cudaMemcpyAsync(ho + r0 * dims.dv, dout + r0 * dims.dv, rows * dims.dv * f,
                           cudaMemcpyDeviceToHost, side->out), "downloading O");
      } else {
        const size_t h0 = c * block_heads, heads = std::min(block_heads, dims.batch - h0);
        ok(cudaMemcpyAsync(dk + h0 * k_floats, hk + h0 * k_floats, heads * k_floats * f,
                           cudaMemcpyHostToDevice, side->in), "uploading K");
        ok(cudaMemcpyAsync(dv + h0 * v_floats, hv + h0 * v_floats, heads * v_floats * f,
                           cudaMemcpyHostToDevice, side->in), "uploading V");
        ok(cudaMemcpyAsync(dq + h0 * q_floats, hq + h0 * q_floats, heads * q_floats * f,
                           cudaMemcpyHostToDevice, side->in), "uploading Q");
        signal(side->in, stream, "ordering a block of heads");
        if (rc == 0)
          rc = ib_attention(dq + h0 * q_floats, dk + h0 * k_floats, dv + h0 * v_floats,
                            dout + h0 * o_floats, heads, dims.nq, dims.nk, dims.d, dims.dv,
                            dims.v_kmajor, precision,
                            choose_geometry(StepKind::Attention, step.hint).kv_granule, ws, ws_bytes,
                            stream);
        signal(stream, side->out, "ordering a download");
        ok(cudaMemcpyAsync(ho + h0 * o_floats, dout + h0 * o_floats, heads * o_floats * f,
                           cudaMemcpyDeviceToHost, side->out), "downloading O");
      }
    }
  }
  // Join both copy streams into `stream` (also after an error: the buffers are
  // freed in `stream` order and must outlive every copy already queued).
  {
    cudaEvent_t a = side->event(), b = side->event();
    if (a && b) {
      cudaEventRecord(a, side->in);
      cudaEventRecord(b, side->out);
      cudaStreamWaitEvent(stream, a, 0);
      cudaStreamWaitEvent(stream, b, 0);
    } else {
      cudaStreamSynchronize(side->in);
      cudaStreamSynchronize(side->out);
    }
  }
  dev.release();
  cudaError_t sync = cudaStreamSynchronize(stream);
  if (rc == 0 && sync != cudaSuccess) {
    set_error(std::string("CUDA error while running the program: ") + cudaGetErrorString(sync));
    rc = -1;
  }
  if (rc == 0) rc = check_device_status("i_exec_into", stream);
  return rc;
}

// Synchronous run accepting host and/or device pointers.
int exec_any(const i_program* program, const i_tensor* inputs, size_t input_count,
             i_tensor_mut* outputs, size_t output_count) {
  const Plan& plan = program->plan;
  std::string err;
  ShapeTable shapes;
  if (!infer_shapes(plan, inputs, input_count, &shapes, &err)) {
    set_error(err);
    return -1;
  }
  if (!device_available(&err)) {
    set_error(err);
    return -1;
  }
  cudaStream_t stream = thread_stream();
  {
    bool all_host = true;
    for (size_t i = 0; i < input_count; ++i) all_host = all_host && !is_device_pointer(inputs[i].data);
    for (size_t o = 0; o < output_count; ++o) all_host = all_host && !is_device_pointer(outputs[o].data);
    if (all_host) {
      const int piped = pipelined_host_attention(program, shapes, inputs, input_count, outputs,
                                                 output_count, stream);
      if (piped <= 0) return piped;
    }
  }
  DeviceBuffers staging;
  staging.stream = stream;
  std::vector<const float*> in_ptrs(input_count);
  std::vector<float*> out_ptrs(output_count);
  std::vector<size_t> out_bytes(output_count);
  int rc = 0;
  for (size_t i = 0; rc == 0 && i < input_count; ++i) {
    const size_t bytes = product(shapes.inputs[i]) * sizeof(float);
    if (bytes && !inputs[i].data) {
      set_error("input " + std::to_string(i) + " has null data");
      rc = -1;
    } else if (bytes == 0 || is_device_pointer(inputs[i].data)) {
      in_ptrs[i] = inputs[i].data;
    } else {
      float* d = staging.alloc(bytes, &err);
      if (!d || cudaMemcpyAsync(d, inputs[i].data, bytes, cudaMemcpyHostToDevice, stream) !=
                    cudaSuccess) {
        set_error(d ? "host to device copy failed" : err);
        rc = -1;
      }
      in_ptrs[i] = d;
    }
  }
  for (size_t o = 0; rc == 0 && o < output_count; ++o) {
    const Source& src = plan.outputs[o];
    const Shape& shape = src.is_input ? shapes.inputs[src.index] : shapes.nodes[src.index];
    out_bytes[o] = product(shape) * sizeof(float);
    if (out_bytes[o] && !outputs[o].data) {
      set_error("output " + std::to_string(o) + " has null data");
      rc = -1;
    } else if (out_bytes[o] == 0 || is_device_pointer(outputs[o].data)) {
      out_ptrs[o] = outputs[o].data;
      out_bytes[o] = 0;  // nothing to copy back
    } else if (!(out_ptrs[o] = staging.alloc(out_bytes[o], &err))) {
      set_error(err);
      rc = -1;
    }
  }
  if (rc == 0) rc = run_plan(program, shapes, in_ptrs.data(), out_ptrs.data(), stream);
  for (size_t o = 0; rc == 0 && o < output_count; ++o)
    if (out_bytes[o] && cudaMemcpyAsync(outputs[o].data, out_ptrs[o], out_bytes[o],
                                        cudaMemcpyDeviceToHost, stream) != cudaSuccess) {
      set_error("device to host copy failed");
      rc = -1;
    }
  staging.release();
  cudaError_t sync = cudaStreamSynchronize(stream);
  if (rc == 0 && sync != cudaSuccess) {
    set_error(std::string("CUDA error while running the program: ") + cudaGetErrorString(sync));
    rc = -1;
  }
  if (rc == 0) rc = check_device_status("i_exec_into", stream);
  return rc;
}

}  // namespace

}  // namespace ib

// ---------------------------------------------------------------------------
// C API
// ---------------------------------------------------------------------------

namespace {

template <typename T>
T* null_with_error(const std::string& message) {
  ib::set_error(message);
  return nullptr;
}

i_component* combine(const i_component* left, const i_component* right, ib::Component::Kind kind) {
  if (!left) return null_with_error<i_component>("null left component");
  if (!right) return null_with_error<i_component>("null right component");
  auto node = std::make_shared<ib::Component>();
  node->kind = kind;
  node->left = left->inner;
  node->right = right->inner;
  return new i_component{node};
}

ib::Result<ib::Plan> plan_component(const i_component* component, ib::Graph* graph_out) {
  ib::Result<ib::Graph> graph = ib::lower_component_to_graph(*component->inner);
  if (!graph.ok()) return ib::Result<ib::Plan>::failure(graph.error.text);
  ib::Result<ib::Plan> plan = ib::make_plan(*graph.value);
  if (plan.ok() && graph_out) *graph_out = std::move(*graph.value);
  return plan;
}

int check_exec_args(const i_program* program, const i_tensor* inputs, size_t input_count,
                    const i_tensor_mut* outputs, size_t output_count) {
  if (!program) return ib::set_error("null program"), -1;
  if (input_count > 0 && !inputs) return ib::set_error("null inputs"), -1;
  if (output_count != program->plan.outputs.size()) return ib::set_error("wrong output count"), -1;
  if (output_count > 0 && !outputs) return ib::set_error("null outputs"), -1;
  return 0;
}

}  // namespace

extern "C" {

i_component* i_parse(const char* src) {
  if (!src) return null_with_error<i_component>("null source");
  ib::Result<ib::Expr> expr = ib::parse_expr(src);
  if (!expr.ok()) return null_with_error<i_component>(expr.error.text);
  auto leaf = std::make_shared<ib::Component>();
  leaf->kind = ib::Component::Leaf;
  leaf->expr = std::move(*expr.value);
  return new i_component{leaf};
}

i_component* i_identity(void) {
  auto node = std::make_shared<ib::Component>();
  node->kind = ib::Component::Identity;
  return new i_component{node};
}

i_component* i_chain(const i_component* l, const i_component* r) {
  return combine(l, r, ib::Component::Chain);
}
i_component* i_compose(const i_component* l, const i_component* r) {
  return combine(l, r, ib::Component::Compose);
}
i_component* i_fanout(const i_component* l, const i_component* r) {
  return combine(l, r, ib::Component::Fanout);
}
i_component* i_pair(const i_component* l, const i_component* r) {
  return combine(l, r, ib::Component::Pair);
}

i_component* i_swap(const i_component* component) {
  if (!component) return null_with_error<i_component>("null component");
  auto node = std::make_shared<ib::Component>();
  node->kind = ib::Component::Swap;
  node->left = component->inner;
  return new i_component{node};
}

char* i_code(const i_component* component) {
  if (!component) return null_with_error<char>("null component");
  ib::Graph graph;
  ib::Result<ib::Plan> plan = plan_component(component, &graph);
  if (!plan.ok()) return null_with_error<char>(plan.error.text);
  std::string text = plan.value->describe() + ib::describe_graph(graph);
  char* out = static_cast<char*>(std::malloc(text.size() + 1));
  if (!out) return null_with_error<char>("out of memory");
  std::memcpy(out, text.c_str(), text.size() + 1);
  return out;
}

i_program* i_compile(const i_component* component) {
  if (!component) return null_with_error<i_program>("null component");
  auto program = new i_program();
  ib::Result<ib::Plan> plan = plan_component(component, &program->graph);
  if (!plan.ok()) {
    delete program;
    return null_with_error<i_program>(plan.error.text);
  }
  program->plan = std::move(*plan.value);
  program->precision.store(ib::default_precision());
  return program;
}

size_t i_output_count(const i_program* program) {
  if (!program) return ib::set_error("null program"), 0;
  return program->plan.outputs.size();
}

int i_output_ranks(const i_program* program, size_t* ranks) {
  if (!program) return ib::set_error("null program"), -1;
  if (!ranks) return ib::set_error("null ranks"), -1;
  const ib::Plan& plan = program->plan;
  for (size_t o = 0; o < plan.outputs.size(); ++o) {
    size_t rank = plan.output_ranks[o];
    if (rank == static_cast<size_t>(-1)) {
      // Output wired straight to an input: its rank is whatever the patterns
      // reading that input say, or 0 if nothing reads it.
      size_t r = plan.input_ranks[plan.outputs[o].index];
      rank = r == static_cast<size_t>(-1) ? 0 : r;
    }
    ranks[o] = rank;
  }
  return 0;
}

int i_output_shapes(const i_program* program, const i_tensor* inputs, size_t input_count,
                    size_t** shapes) {
  if (!program) return ib::set_error("null program"), -1;
  if (input_count > 0 && !inputs) return ib::set_error("null inputs"), -1;
  if (!shapes) return ib::set_error("null shapes"), -1;
  ib::ShapeTable table;
  std::string err;
  if (!ib::infer_shapes(program->plan, inputs, input_count, &table, &err))
    return ib::set_error(err), -1;
  const ib::Plan& plan = program->plan;
  for (size_t o = 0; o < plan.outputs.size(); ++o) {
    const ib::Source& src = plan.outputs[o];
    const ib::Shape& shape = src.is_input ? table.inputs[src.index] : table.nodes[src.index];
    for (size_t d = 0; d < shape.size(); ++d) shapes[o][d] = shape[d];
  }
  return 0;
}

int i_exec_into(const i_program* program, const i_tensor* inputs, size_t input_count,
                i_tensor_mut* outputs, size_t output_count) {
  if (int rc = check_exec_args(program, inputs, input_count, outputs, output_count)) return rc;
  return ib::exec_any(program, inputs, input_count, outputs, output_count);
}

int i_b200_exec_into(const i_program* program, const i_tensor* inputs, size_t input_count,
                     i_tensor_mut* outputs, size_t output_count, void* stream) {
  if (int rc = check_exec_args(program, inputs, input_count, outputs, output_count)) return rc;
  std::string err;
  ib::ShapeTable shapes;
  if (!ib::infer_shapes(program->plan, inputs, input_count, &shapes, &err))
    return ib::set_error(err), -1;
  if (!ib::device_available(&err)) return ib::set_error(err), -1;
  // A wait that timed out in an earlier asynchronous launch is reported here.
  if (int rc = ib::check_device_status("i_b200_exec_into (earlier launch)", nullptr)) return rc;
  std::vector<const float*> in_ptrs(input_count);
  std::vector<float*> out_ptrs(output_count);
  for (size_t i = 0; i < input_count; ++i) in_ptrs[i] = inputs[i].data;
  for (size_t o = 0; o < output_count; ++o) out_ptrs[o] = outputs[o].data;
  return ib::run_plan(program, shapes, in_ptrs.data(), out_ptrs.data(),
                      static_cast<cudaStream_t>(stream));
}

i_outputs i_exec(const i_program* program, const i_tensor* inputs, size_t input_count) {
  i_outputs none{nullptr, 0};
  if (!program) return ib::set_error("null program"), none;
  if (input_count > 0 && !inputs) return ib::set_error("null inputs"), none;
  ib::ShapeTable table;
  std::string err;
  if (!ib::infer_shapes(program->plan, inputs, input_count, &table, &err))
    return ib::set_error(err), none;
  const ib::Plan& plan = program->plan;
  const size_t count = plan.outputs.size();
  i_owned_tensor* tensors =
      static_cast<i_owned_tensor*>(std::calloc(count ? count : 1, sizeof(i_owned_tensor)));
  std::vector<i_tensor_mut> views(count);
  bool ok = tensors != nullptr;
  for (size_t o = 0; ok && o < count; ++o) {
    const ib::Source& src = plan.outputs[o];
    const ib::Shape& shape = src.is_input ? table.inputs[src.index] : table.nodes[src.index];
    i_owned_tensor& t = tensors[o];
    t.rank = shape.size();
    t.len = ib::product(shape);
    t.shape = static_cast<size_t*>(std::malloc((t.rank ? t.rank : 1) * sizeof(size_t)));
    t.data = static_cast<float*>(std::calloc(t.len ? t.len : 1, sizeof(float)));
    ok = t.shape && t.data;
    if (ok) std::copy(shape.begin(), shape.end(), t.shape);
    views[o] = i_tensor_mut{t.data, t.shape, t.rank};
  }
  i_outputs result{tensors, count};
  if (!ok) ib::set_error("out of memory");
  if (!ok || ib::exec_any(program, inputs, input_count, views.data(), count) != 0) {
    i_outputs_free(result);
    return none;
  }
  return result;
}

const char* i_error(void) { return ib::g_has_error ? ib::g_error.c_str() : nullptr; }

void i_component_free(i_component* component) { delete component; }
void i_program_free(i_program* program) { delete program; }

void i_outputs_free(i_outputs outputs) {
  if (!outputs.tensors) return;
  for (size_t o = 0; o < outputs.count; ++o) {
    std::free(outputs.tensors[o].data);
    std::free(outputs.tensors[o].shape);
  }
  std::free(outputs.tensors);
}

void i_string_free(char* s) { std::free(s); }

int i_b200_program_set_precision(i_program* program, int precision) {
  if (!program) return ib::set_error("null program"), -1;
  if (precision < IB_PRECISION_AUTO || precision > IB_PRECISION_F16)
    return ib::set_error("unknown precision"), -1;
  program->precision.store(precision);
  return 0;
}

int i_b200_program_precision(const i_program* program) {
  if (!program) return ib::set_error("null program"), -1;
  return program->precision.load();
}

int i_b200_device_count(void) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return count;
}

size_t i_b200_launch_count(void) { return ib::g_launches.load(); }

}  // extern "C"
