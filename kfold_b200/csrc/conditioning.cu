// Small pieces of the sampler's single conditioning (noise-level embedding and its broadcast onto the tokens).
// Both are tiny: a handful of rows per sampler step.  They exist so that the conditioning never leaves the library.
#include <cuda_bf16.h>

#include "ops_common.cuh"

namespace kfb {
namespace {

// out[row][j] = cos(2 pi t[row] w[j] + b[j]): the random Fourier features of the noise level.  The argument is
// reduced exactly by cospif (cos(pi x) with x = 2 t w + b / pi), so large |t w| loses nothing to range reduction.
__global__ void __launch_bounds__(256) fourier_embed_kernel(const float* __restrict__ t, const float* __restrict__ w,
                                                            const float* __restrict__ b, float* __restrict__ out, int rows, int dim) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * dim) return;
  const int row = idx / dim, j = idx - row * dim;
  const float x = 2.0f * t[row] * w[j];
  out[idx] = cospif(x + b[j] * 0.31830988618379067f);
}

// out[g][n][l][:] = s[g][l][:] + f[g][n][:]   (token conditioning plus the per-sample noise embedding), fp32
__global__ void __launch_bounds__(256) broadcast_add_kernel(const float* __restrict__ s, const float* __restrict__ f,
                                                            float* __restrict__ out, long long total, int samples, int l, int c) {
  const long long idx = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (idx >= total) return;
  const int col = static_cast<int>(idx % c);
  const long long row = idx / c;                       // (g, n, l)
  const int li = static_cast<int>(row % l);
  const long long gn = row / l;                        // g * samples + n
  const long long g = gn / samples;
  const float4 a = *reinterpret_cast<const float4*>(s + (g * l + li) * c + col);
  const float4 e = *reinterpret_cast<const float4*>(f + gn * c + col);
  *reinterpret_cast<float4*>(out + idx) = make_float4(a.x + e.x, a.y + e.y, a.z + e.z, a.w + e.w);
}

}  // namespace
}  // namespace kfb

using namespace kfb;

extern "C" {

KFB_API int kfb_fourier_embed(const float* t, const float* w, const float* b, float* out, int rows, int dim, void* stream_) {
  KFB_CHECK_ARG(t && w && b && out, "fourier_embed: null pointer");
  KFB_CHECK_ARG(rows >= 1 && dim >= 1 && static_cast<long long>(rows) * dim < (1ll << 31), "fourier_embed: rows %d dim %d", rows, dim);
  cudaStream_t stream = as_stream(stream_);
  LaunchScope scope(stream, "fourier_embed");
  fourier_embed_kernel<<<cdiv(rows * dim, 256), 256, 0, stream>>>(t, w, b, out, rows, dim);
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

KFB_API int kfb_broadcast_add(const float* s, const float* f, float* out, int groups, int samples, int l, int c, void* stream_) {
  KFB_CHECK_ARG(s && f && out, "broadcast_add: null pointer");
  KFB_CHECK_ARG(groups >= 1 && samples >= 1 && l >= 1 && c >= 4 && c % 4 == 0, "broadcast_add: groups %d samples %d l %d c %d",
                groups, samples, l, c);
  KFB_CHECK_ARG(((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(f) | reinterpret_cast<uintptr_t>(out)) & 15) == 0,
                "broadcast_add: pointers must be 16-byte aligned");
  cudaStream_t stream = as_stream(stream_);
  const long long total = static_cast<long long>(groups) * samples * l * c;
  LaunchScope scope(stream, "broadcast_add");
  broadcast_add_kernel<<<static_cast<unsigned>((total / 4 + 255) / 256), 256, 0, stream>>>(s, f, out, total, samples, l, c);
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

}  // extern "C"
