// Token <-> atom maps around the atom transformers: a row gather (token features broadcast to their atoms) and a
// masked mean over the atoms of every token.  Both are pure data movement, HBM/L2-bound and tiny next to the
// transformers; they exist so that a caller never has to leave the library between the atom and the token level.
#include <cuda_bf16.h>

#include "ops_common.cuh"
#include "ptx.cuh"

namespace kfb {
namespace {

__device__ __forceinline__ float ld_f(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float ld_f(const float* p) { return *p; }
__device__ __forceinline__ void st_f(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void st_f(float* p, float v) { *p = v; }

// out[b][a][:] = x[b][index[b / index_div][a]][:]; one warp per atom row, 16-byte pieces.  An index outside
// [0, n_token) yields a zero row and records code 900 in the device status word instead of reading out of bounds.
static constexpr int kBadIndexCode = 900;
template <typename T>
__global__ void __launch_bounds__(256) tokens_to_atoms_kernel(const T* __restrict__ x, const long long* __restrict__ index,
                                                              T* __restrict__ out, long long rows, int n_atom, int n_token, int d,
                                                              int index_div) {
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long b = row / n_atom;
  const int a = static_cast<int>(row - b * n_atom);
  const long long t = index[(b / index_div) * n_atom + a];
  const bool ok = t >= 0 && t < n_token;
  if (!ok && lane == 0) atomicCAS(&g_status, 0, kBadIndexCode);
  constexpr int kVec = 16 / sizeof(T);
  const T* src = x + (b * n_token + (ok ? t : 0)) * d;
  T* dst = out + row * d;
  if (d % kVec == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
    for (int i = lane * kVec; i < d; i += 32 * kVec)
      *reinterpret_cast<uint4*>(dst + i) = ok ? *reinterpret_cast<const uint4*>(src + i) : make_uint4(0, 0, 0, 0);
  } else {
    for (int i = lane; i < d; i += 32) st_f(dst + i, ok ? ld_f(src + i) : 0.f);
  }
}

// out[b][t][:] = mean over the atoms a of batch entry b with mask[a] and index[a] == t of x[b][a][:] (0 for a token
// without atoms).  One warp per (b, t): the warp scans the atom indices 32 at a time and adds the matching rows in
// atom order with fp32 accumulators, so the result does not depend on scheduling.  kChunks * 32 channels per pass.
template <typename T, int kChunks>
__global__ void __launch_bounds__(256) atoms_to_tokens_kernel(const T* __restrict__ x, const long long* __restrict__ index,
                                                              const unsigned char* __restrict__ mask, T* __restrict__ out,
                                                              long long rows, int n_atom, int n_token, int d, int index_div) {
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long b = row / n_token;
  const int t = static_cast<int>(row - b * n_token);
  const long long* idx = index + (b / index_div) * n_atom;
  const unsigned char* mk = mask + (b / index_div) * n_atom;
  const T* xb = x + b * n_atom * d;
  for (int d0 = 0; d0 < d; d0 += kChunks * 32) {
    float acc[kChunks];
#pragma unroll
    for (int k = 0; k < kChunks; ++k) acc[k] = 0.f;
    int count = 0;
    for (int a0 = 0; a0 < n_atom; a0 += 32) {
      const int a = a0 + lane;
      const bool hit = a < n_atom && mk[a] != 0 && idx[a] == t;
      unsigned m = __ballot_sync(0xffffffffu, hit);
      count += __popc(m);
      while (m) {
        const int j = __ffs(m) - 1;
        m &= m - 1;
        const T* src = xb + static_cast<long long>(a0 + j) * d + d0;
#pragma unroll
        for (int k = 0; k < kChunks; ++k) {
          const int col = k * 32 + lane;
          if (d0 + col < d) acc[k] += ld_f(src + col);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < kChunks; ++k) {
      const int col = d0 + k * 32 + lane;
      // the reference divides the sum by the count (scatter_reduce "mean"): a division, not a multiplication
      if (col < d) st_f(out + row * d + col, count > 0 ? acc[k] / static_cast<float>(count) : 0.f);
    }
  }
}

}  // namespace
}  // namespace kfb

using namespace kfb;

extern "C" {

KFB_API int kfb_tokens_to_atoms(const void* x, const long long* token_index, void* out, int batch, int n_token, int n_atom,
                                int d, int index_div, int dtype, void* stream_) {
  KFB_CHECK_ARG(x && token_index && out, "tokens_to_atoms: null pointer");
  KFB_CHECK_ARG(dtype == KFB_BF16 || dtype == KFB_FP32, "tokens_to_atoms: dtype %d (bf16 or fp32)", dtype);
  KFB_CHECK_ARG(batch >= 1 && n_token >= 1 && n_atom >= 1 && d >= 1 && index_div >= 1 && batch % index_div == 0,
                "tokens_to_atoms: batch %d tokens %d atoms %d d %d index_div %d", batch, n_token, n_atom, d, index_div);
  cudaStream_t stream = as_stream(stream_);
  const long long rows = static_cast<long long>(batch) * n_atom;
  const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
  LaunchScope scope(stream, "tokens_to_atoms");
  if (dtype == KFB_BF16)
    tokens_to_atoms_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), token_index,
                                                                       static_cast<__nv_bfloat16*>(out), rows, n_atom, n_token, d,
                                                                       index_div);
  else
    tokens_to_atoms_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(x), token_index, static_cast<float*>(out),
                                                               rows, n_atom, n_token, d, index_div);
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

KFB_API int kfb_atoms_to_tokens(const void* x, const long long* token_index, const unsigned char* mask, void* out, int batch,
                                int n_atom, int n_token, int d, int index_div, int dtype, void* stream_) {
  KFB_CHECK_ARG(x && token_index && mask && out, "atoms_to_tokens: null pointer");
  KFB_CHECK_ARG(dtype == KFB_BF16 || dtype == KFB_FP32, "atoms_to_tokens: dtype %d (bf16 or fp32)", dtype);
  KFB_CHECK_ARG(batch >= 1 && n_token >= 1 && n_atom >= 1 && d >= 1 && index_div >= 1 && batch % index_div == 0,
                "atoms_to_tokens: batch %d tokens %d atoms %d d %d index_div %d", batch, n_token, n_atom, d, index_div);
  cudaStream_t stream = as_stream(stream_);
  const long long rows = static_cast<long long>(batch) * n_token;
  const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
  LaunchScope scope(stream, "atoms_to_tokens");
  if (dtype == KFB_BF16)
    atoms_to_tokens_kernel<__nv_bfloat16, 8><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), token_index, mask,
                                                                          static_cast<__nv_bfloat16*>(out), rows, n_atom, n_token, d,
                                                                          index_div);
  else
    atoms_to_tokens_kernel<float, 8><<<blocks, 256, 0, stream>>>(static_cast<const float*>(x), token_index, mask,
                                                                  static_cast<float*>(out), rows, n_atom, n_token, d, index_div);
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

}  // extern "C"
