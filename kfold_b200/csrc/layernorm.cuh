// HBM-bound normalisation kernels (declarations).
#pragma once
#include "common.cuh"

namespace kfb {

// Row-wise LayerNorm, one warp per row, fp32 statistics.  in/out dtype KFB_BF16 or KFB_FP32.
int launch_layernorm(cudaStream_t stream, const void* x, void* y, const float* w, const float* b, long long rows, int c,
                     long long xs, long long ys, float eps, int in_dtype, int out_dtype);

// LayerNorm over channels of a CHANNEL-major tensor t[batch][c][pos] (pos contiguous, channel stride
// `chan_stride`, batch stride `batch_stride`), written POSITION-major y[batch*npos + pos][c] in bf16.
// `in_dtype` is the element type of t.  Used on the triangle contraction's output.
int launch_layernorm_cm(cudaStream_t stream, const void* t, __nv_bfloat16* y, const float* w, const float* b, int batch,
                        long long npos, int c, long long chan_stride, long long batch_stride, float eps, int in_dtype);

// Adaptive LayerNorm: y[r] = sigmoid(g[s(r)]) * LN(a[r]) + v[s(r)], LN without affine, fp32 statistics.
// a, y: `rows` rows of c channels; gv: rows_s rows of [2c] (gate logits | shift), bf16.  Row r of a uses row
// (r / (samples * l)) * l + r % l of gv: the conditioning is shared by the `samples` diffusion samples.
int launch_adaln(cudaStream_t stream, const void* a, void* y, const __nv_bfloat16* gv, long long rows, int c, int samples,
                 int l, float eps, int in_dtype, int out_dtype);

}  // namespace kfb
