// Internal interfaces between the kernel translation units.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>

#include "i_b200.h"

namespace ib {

// contract_simt.cu
// With splits > 1 the k range is cut into that many parts and c receives one copy of the result
// per part, [batch][split][m][n], for the caller to add (sum_partials in reduce.cu).
int contract_simt(const float* a, const float* b, float* c, size_t batch, size_t m, size_t n,
                  size_t k, bool a_kmajor, bool b_kmajor, cudaStream_t s, size_t splits = 1);
// y[b][c] = sum_r x[b][r][c] for a handful of rows (the copies of a split contraction).
int sum_partials(const float* x, float* y, size_t batch, size_t rows, size_t cols, cudaStream_t s);
// out[b][c][r] = in[b][r][c]; rows of `out` are `out_pitch` elements apart.  With
// `round` the values are rounded to TF32 (nearest) on the way.
int transpose_batched(const float* in, float* out, size_t batch, size_t rows, size_t cols,
                      size_t out_pitch, bool round, cudaStream_t s);
// Rounds one or two row-major arrays to TF32 (nearest) in a single launch; pass
// in1 = nullptr for one.  Pitches are in elements.
int round_tf32_rows(const float* in0, float* out0, size_t rows0, size_t cols0, size_t in_pitch0,
                    size_t out_pitch0, const float* in1, float* out1, size_t rows1, size_t cols1,
                    size_t in_pitch1, size_t out_pitch1, cudaStream_t s);

// One launch: qr = round_tf32(q), kr = round_tf32(k) (element counts multiples
// of 4, 16-byte aligned), vt[b][c][r] = round_tf32(v[b][r][c]) with row pitch `pitch`.
int prepare_attention_operands(const float* q, float* qr, size_t q_elems, const float* k,
                               float* kr, size_t k_elems, const float* v, float* vt, size_t batch,
                               size_t nk, size_t dv, size_t pitch, cudaStream_t s);

// reduce.cu — y[r] = sum_c x[r][c] * w[r][c], or x[r][c] * w[c] with w_is_vector: row-wise dot
// products and matrix times vector as one pass over memory (products rounded, then a tree sum).
// Few rows of very many columns are folded in segments; `partials` then holds long_rows_floats
// floats (null: every row is folded whole).
size_t long_rows_floats(size_t rows, size_t cols);
int dot_rows(const float* x, const float* w, bool w_is_vector, float* y, size_t rows, size_t cols,
             cudaStream_t s, float* partials = nullptr);
// y[c] = sum_r x[r][c] * w[r] (vector times matrix); `partials` holds dot_leading_axis_floats
// floats (null: the rows are folded as one slab).
size_t dot_leading_axis_floats(size_t rows, size_t cols);
int dot_leading_axis(const float* x, const float* w, float* y, size_t rows, size_t cols,
                     float* partials, cudaStream_t s);

// device_util.cu — encodes a TMA descriptor for a dense fp32 tensor
// [batch][rows][cols] (cols contiguous, `row_pitch` elements between rows) read
// in boxes of 32 columns (128 bytes, 128-byte swizzle) x box_rows rows.
// Returns 0, or -1 with the error recorded.
int make_tensor_map_f32(CUtensorMap* map, const float* base, size_t batch, size_t rows,
                        size_t cols, size_t row_pitch, size_t batch_pitch, unsigned box_rows);

// Same for a bf16 tensor, boxes of 64 columns (128 bytes).
int make_tensor_map_bf16(CUtensorMap* map, const void* base, size_t batch, size_t rows,
                         size_t cols, size_t row_pitch, size_t batch_pitch, unsigned box_rows);

// Per-launch status word the tcgen05 kernels report bounded-wait timeouts into.
// Lives in device memory owned by the library; zeroed before each launch that
// uses it and read back only on demand.
int* device_status_word(cudaStream_t s);
int check_device_status(const char* what, cudaStream_t s);

// gemm_tcgen05.cu — C[b][i][j] = sum_k A[b][i][k] B[b][j][k], both operands
// K-major fp32 fed to tcgen05 kind::tf32.
bool gemm_tcgen05_supported(const float* a, const float* b, const float* c, size_t m, size_t n,
                            size_t k);
// Tile geometry a caller may fix (zeros = the kernel's own choice): output columns per tile (128 or
// 256), and how many column tiles form a group that is walked over all row tiles before the next
// group (1 = column by column, at least the number of column tiles = row by row; default 12).
struct GemmGeometry {
  int col_tile = 0;
  int group_n = 0;
};
// Pointwise operators the tensor-core contraction applies to every element of its result before
// storing it (a bias, a rectifier, a scale), in order: acc = op(acc, other), op(other, acc) with
// acc_right, or the one-operand form op(acc) with which < 0.  `other` is operand[which], addressed
// by mode 0 [row][col] (the result's own shape, batch entries flattened into rows), 1 [row],
// 2 [col], 3 one value.  Operators: IB_OP_ADD, IB_OP_SUB, IB_OP_MUL, IB_OP_MAX, IB_OP_MIN, with
// the arithmetic of the pointwise kernels, so the result equals contraction then maps bit for bit.
struct GemmEpilogue {
  int n_ops = 0;
  int op[IB_MAX_CHAIN_OPS] = {};
  int which[IB_MAX_CHAIN_OPS] = {};
  int acc_right[IB_MAX_CHAIN_OPS] = {};
  const float* operand[IB_MAX_CHAIN_OPERANDS] = {};
  int mode[IB_MAX_CHAIN_OPERANDS] = {};
};
// k_parts > 1 (one batch entry, k a multiple of 4 * k_parts): the k range is cut into that many
// equal parts and c receives one copy of the result per part, [part][m][n], for the caller to add.
int gemm_tcgen05(const float* a, const float* b, float* c, size_t batch, size_t m, size_t n,
                 size_t k, cudaStream_t s, GemmGeometry g = {}, const GemmEpilogue* e = nullptr,
                 size_t k_parts = 1);
// Same contraction with bf16 operands a16 / b16 ([b][rows][k_pitch] bf16, k_pitch a multiple of 8)
// fed to tcgen05 kind::f16, fp32 accumulation.
// The same on fp16 operands stored over one power of two per row (a16[b][i][:] = A / a_scale[b][i],
// b16 likewise): the epilogue multiplies the two scales back, so the result carries TF32's rounding
// at the 16-bit issue rate.
int gemm_tcgen05_f16(const void* a16, const void* b16, const float* a_scale, const float* b_scale,
                     float* c, size_t batch, size_t m, size_t n, size_t k, size_t k_pitch,
                     cudaStream_t s, GemmGeometry g = {}, const GemmEpilogue* e = nullptr);
int gemm_tcgen05_bf16(const void* a16, const void* b16, float* c, size_t batch, size_t m, size_t n,
                      size_t k, size_t k_pitch, cudaStream_t s, GemmGeometry g = {},
                      const GemmEpilogue* e = nullptr);
// out[r][c] = bf16(in[r][c]) (round to nearest even) for a [rows][cols] fp32 array; `out_pitch` in
// elements, columns cols..out_pitch-1 are zeroed.
// fp16 rows over one power of two each: out[r][c] = fp16(in[r][c] / scale[r]), scale[r] bringing the
// row's largest magnitude into [2^14, 2^15); out_pitch % 8 == 0, pad columns zero.
int convert_f16_rows_scaled(const float* in, void* out, float* scale, size_t rows, size_t cols,
                            size_t out_pitch, cudaStream_t s);
int convert_bf16_rows(const float* in, void* out, size_t rows, size_t cols, size_t out_pitch,
                      cudaStream_t s);

// attention_tcgen05.cu — fused online-softmax attention; q is the caller's fp32
// Q, k a TF32-rounded copy of K, vt the rounded V transposed to [b][dv][nk_pitch].
// Floats of scratch for the partial results of row tiles shared between CTAs.
size_t attention_tcgen05_partial_floats(size_t batch, size_t nq, size_t nk, size_t dv,
                                        int* ctas_out);
// Operand types: TF32 — k, vt fp32 rounded to TF32 ([b][nk][d], [b][dv][nk_pitch], pitch % 4 == 0);
// BF16 — both bf16 ([b][nk][d_pitch], [b][dv][nk_pitch], pitches % 8 == 0), kind::f16 MMAs;
// MIXED — k as in TF32, vt fp16 holding V / v_scale[head] (nk_pitch % 8 == 0): S = Q K^T in TF32,
// O += P V in fp16 (same 10-bit mantissa); F16 — k fp16 holding K / k_tile_scale[head][key / 128]
// ([b][nk][d_pitch], d_pitch % 8 == 0), vt as in MIXED: both contractions in fp16.  follows_prepare: the kernel before this call in the
// stream is the one that wrote k and vt (the launch may then overlap its tail).  logit_scale: one
// float on the device, or null; the logits are S * it, or S / it with logit_divide.  kv_granule:
// a row tile's key range is divided between CTAs only at multiples of this many keys (rounded up
// to whole 128-key tiles; 0 = one tile); nk or more = never divided, and no merge kernel runs.
enum class AttentionArm { TF32, BF16, MIXED, F16 };
int attention_tcgen05(const float* q, const void* k, const void* vt, float* o, size_t batch,
                      size_t nq, size_t nk, size_t d, size_t dv, size_t d_pitch, size_t nk_pitch,
                      AttentionArm arm, const float* v_scale, const float* k_tile_scale,
                      const float* logit_scale, bool logit_divide, bool follows_prepare,
                      float* partials, size_t kv_granule, cudaStream_t s);
// Mixed-arm operand preparation: kr = K rounded to TF32; vt16[b][c][nk_pitch] = fp16(V^T / scale[b])
// with scale[b] the power of two that brings the head's largest |V| into [2^14, 2^15); block_max
// is scratch of batch * kAbsmaxBlocks floats.
constexpr int kAbsmaxBlocks = 256;   // partial maxima per head (= threads of the block that folds them)
int prepare_attention_operands_mixed(const float* k, float* kr, const float* v, void* vt16,
                                     float* scale, float* block_max, size_t batch, size_t nk,
                                     size_t d, size_t dv, size_t nk_pitch, bool v_kmajor,
                                     cudaStream_t s);
// bf16 operand preparation: k16[b][r][d_pitch] = bf16(k), vt16[b][c][nk_pitch] = bf16(v^T);
// pad columns are zeroed.
// fp16-arm operand preparation: k16[b][key][d_pitch] = fp16(K / k_tile_scale[b][key / 128]), every
// tile of 128 keys over the power of two that brings its largest |K| into [2^14, 2^15); V as in
// the mixed arm.
int prepare_attention_operands_f16(const float* k, void* k16, float* k_tile_scale, const float* v,
                                   void* vt16, float* v_scale, float* block_max, size_t batch,
                                   size_t nk, size_t d, size_t dv, size_t d_pitch, size_t nk_pitch,
                                   bool v_kmajor, cudaStream_t s);
int prepare_attention_operands_bf16(const float* k, void* k16, const float* v, void* vt16,
                                    size_t batch, size_t nk, size_t d, size_t dv, size_t d_pitch,
                                    size_t nk_pitch, bool v_kmajor, cudaStream_t s);

void set_attention_profile(unsigned long long* device_counters);
void set_reserved_sms(int n);
int reserved_sms();

}  // namespace ib
