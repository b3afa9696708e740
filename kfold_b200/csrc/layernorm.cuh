// HBM-bound normalisation kernels (declarations).
#pragma once
#include "common.cuh"

namespace kfb {

// Output row order of a (rows, n) shard written as the send buffer of a shard transpose: row (i, q * rows + j) goes to
// block q, [q][i][j].  rows == 0: rows keep their order.
struct RowPerm {
  int rows = 0;
  int n = 0;
};

// Row-wise LayerNorm, one warp per row, fp32 statistics.  in/out dtype KFB_BF16 or KFB_FP32.
int launch_layernorm(cudaStream_t stream, const void* x, void* y, const float* w, const float* b, long long rows, int c,
                     long long xs, long long ys, float eps, int in_dtype, int out_dtype, RowPerm perm = RowPerm());

// Row-wise LayerNorm of fp32 rows written as the bf16 triple split [x0 x0 x1 x1 x0 x2] (six blocks of c columns,
// row stride 6c): the A operand of the fp32-accurate GEMMs.  With w == b == nullptr and `normalise` == 0 it only
// splits (used for operands that are not normalised).
int launch_layernorm_split(cudaStream_t stream, const float* x, __nv_bfloat16* y6, const float* w, const float* b, long long rows,
                           int c, long long xs, float eps, int normalise);

// LayerNorm over channels of a CHANNEL-major tensor t[batch][c][pos] (pos contiguous, channel stride
// `chan_stride`, batch stride `batch_stride`), written POSITION-major y[batch*npos + pos][c] in bf16.
// `in_dtype` is the element type of t.  Used on the triangle contraction's output.
int launch_layernorm_cm(cudaStream_t stream, const void* t, __nv_bfloat16* y, const float* w, const float* b, int batch,
                        long long npos, int c, long long chan_stride, long long batch_stride, float eps, int in_dtype,
                        int split_out = 0);  // split_out: y is the [x0 x0 x1 x1 x0 x2] split, row stride 6c

// Adaptive LayerNorm: y[r] = sigmoid(g[s(r)]) * LN(a[r]) + v[s(r)], LN without affine, fp32 statistics.
// a, y: `rows` rows of c channels; gv: rows_s rows of [2c] (gate logits | shift), bf16.  Row r of a uses row
// (r / (samples * l)) * l + r % l of gv: the conditioning is shared by the `samples` diffusion samples.
// gv_ld: elements between consecutive gv rows (0 = 2c), for rows that are slices of a wider table.
int launch_adaln(cudaStream_t stream, const void* a, void* y, const void* gv, long long rows, int c, int samples,
                 int l, float eps, int in_dtype, int out_dtype, long long gv_ld = 0);

// LayerNorm folded into the following GEMM (see layernorm.cu): per-position (mean, rstd) of a channel-major tensor, and the
// folded weights W' = gamma * W (bf16) with s1[n] = sum_k W'[n][k], s0[n] = sum_k beta[k] W[n][k].
int launch_cm_stats(cudaStream_t stream, const __nv_bfloat16* t, float2* stats, long long npos, int c, long long chan_stride,
                    float eps);
int launch_ln_fold_weights(cudaStream_t stream, const __nv_bfloat16* w, const float* gamma, const float* beta, __nv_bfloat16* wf,
                           float* s1, float* s0, int n, int k);

// LayerNorm over c (16, 32 or 64) channels and projection to nh values per position: x [npos][c], w [nh][c] of `dtype`
// (KFB_BF16 or KFB_FP32), y [nh][npos] of the same type.  normalise == 0: projection only.
int launch_window_bias(cudaStream_t stream, const void* x, const float* ln_w, const float* ln_b, const void* w, void* y,
                       long long npos, int c, int nh, float eps, int normalise, int dtype);

}  // namespace kfb
