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
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// out[b][a][:] = x[b][index[b / index_div][a]][:] (+ addend[b][a][:]); one warp per atom row, 16-byte pieces when the
// types agree and nothing is added.  An index outside [0, n_token) yields a zero row (plus the addend) and records
// code 900 in the device status word instead of reading out of bounds.
static constexpr int kBadIndexCode = 900;
template <typename TX, typename TO>
__global__ void __launch_bounds__(256) tokens_to_atoms_kernel(const TX* __restrict__ x, const long long* __restrict__ index,
                                                              const TO* __restrict__ addend, TO* __restrict__ out, long long rows,
                                                              int n_atom, int n_token, int d, int index_div) {
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long b = row / n_atom;
  const int a = static_cast<int>(row - b * n_atom);
  const long long t = index[(b / index_div) * n_atom + a];
  const bool ok = t >= 0 && t < n_token;
  if (!ok && lane == 0) atomicCAS(&g_data_status, 0, kBadIndexCode);
  const TX* src = x + (b * n_token + (ok ? t : 0)) * d;
  TO* dst = out + row * d;
  if constexpr (sizeof(TX) == sizeof(TO)) {
    constexpr int kVec = 16 / sizeof(TX);
    if (addend == nullptr && d % kVec == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
      for (int i = lane * kVec; i < d; i += 32 * kVec)
        *reinterpret_cast<uint4*>(dst + i) = ok ? *reinterpret_cast<const uint4*>(src + i) : make_uint4(0, 0, 0, 0);
      return;
    }
  }
  const TO* add = addend == nullptr ? nullptr : addend + row * d;
  for (int i = lane; i < d; i += 32) st_f(dst + i, (ok ? ld_f(src + i) : 0.f) + (add != nullptr ? ld_f(add + i) : 0.f));
}

// out[row][:] = q[qrow][:] + sum_k w[:, k] r[row][k], fp32 out: the coordinate embedding added to the atom features
// (row r of out uses row (r / (samples * l)) * l + r % l of q and of the optional atom mask: the samples share them).
// One warp per row.
template <typename TQ>
__global__ void __launch_bounds__(256) coord_embed_kernel(const TQ* __restrict__ q, const float* __restrict__ r,
                                                          const float* __restrict__ w, const unsigned char* __restrict__ mask,
                                                          float* __restrict__ out, long long rows, int c, int kc, int samples, int l) {
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long qrow = (row / (static_cast<long long>(samples) * l)) * l + row % l;
  float rv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const bool keep = mask == nullptr || mask[qrow] != 0;   // coordinates of padding atoms count as zero
  for (int k = 0; k < kc; ++k) rv[k] = keep ? r[row * kc + k] : 0.f;
  for (int i = lane; i < c; i += 32) {
    float acc = 0.f;
    for (int k = 0; k < kc; ++k) acc = fmaf(rv[k], w[i * kc + k], acc);   // same order as a dot product over k
    out[row * c + i] = ld_f(q + qrow * c + i) + acc;
  }
}

// out[row][j] = sum_i LayerNorm(x[row])[i] w[j][i], j < n_out <= 8, everything fp32 after the load: the projection of the
// atom features to coordinate updates.  One warp per row; the row is re-read from L1 for the three passes.
template <typename T>
__global__ void __launch_bounds__(256) ln_project_kernel(const T* __restrict__ x, const float* __restrict__ ln_w,
                                                         const float* __restrict__ ln_b, const float* __restrict__ w,
                                                         const unsigned char* __restrict__ mask, float* __restrict__ out,
                                                         long long rows, int c, int n_out, float eps, int samples, int l) {
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  if (mask != nullptr && mask[(row / (static_cast<long long>(samples) * l)) * l + row % l] == 0) {
    if (lane < n_out) out[row * n_out + lane] = 0.f;   // padding atoms get a zero update
    return;
  }
  const T* xr = x + row * c;
  float s = 0.f;
  for (int i = lane; i < c; i += 32) s += ld_f(xr + i);
  const float mean = warp_sum(s) / static_cast<float>(c);
  float q = 0.f;
  for (int i = lane; i < c; i += 32) {
    const float dlt = ld_f(xr + i) - mean;
    q += dlt * dlt;
  }
  const float rstd = rsqrtf(warp_sum(q) / static_cast<float>(c) + eps);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int i = lane; i < c; i += 32) {
    const float xn = (ld_f(xr + i) - mean) * rstd * (ln_w != nullptr ? ln_w[i] : 1.f) + (ln_b != nullptr ? ln_b[i] : 0.f);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < n_out) acc[j] = fmaf(xn, w[j * c + i], acc[j]);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (j < n_out) {
      const float v = warp_sum(acc[j]);
      if (lane == 0) out[row * n_out + j] = v;
    }
  }
}

// Per (index row, token): the first and last valid atom that maps to the token (first > last: none).  The mean below
// then scans only that range; it still tests every atom in it, so unsorted indices stay correct, and for the usual
// sorted atom order the range is just the token's own atoms.
__global__ void __launch_bounds__(256) token_range_init_kernel(int2* __restrict__ range, long long n) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) range[i] = make_int2(0x7fffffff, -1);
}
__global__ void __launch_bounds__(256) token_range_kernel(const long long* __restrict__ index, const unsigned char* __restrict__ mask,
                                                          int2* __restrict__ range, long long total, int n_atom, int n_token) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = index[i];
  if (mask[i] == 0 || t < 0 || t >= n_token) return;
  const long long row = i / n_atom;
  const int a = static_cast<int>(i - row * n_atom);
  int* r = reinterpret_cast<int*>(range + row * n_token + t);
  atomicMin(r, a);
  atomicMax(r + 1, a);
}

// out[b][t][:] = mean over the atoms a of batch entry b with mask[a] and index[a] == t of x[b][a][:] (0 for a token
// without atoms); with `relu` the features pass through max(., 0) first.  One warp per (b, t): the warp scans the atom indices 32 at a time and adds the matching rows in
// atom order with fp32 accumulators, so the result does not depend on scheduling.  kChunks * 32 channels per pass.
template <typename T, int kChunks>
__global__ void __launch_bounds__(256) atoms_to_tokens_kernel(const T* __restrict__ x, const long long* __restrict__ index,
                                                              const unsigned char* __restrict__ mask, T* __restrict__ out,
                                                              long long rows, int n_atom, int n_token, int d, int index_div,
                                                              int relu, const int2* __restrict__ range) {
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long b = row / n_token;
  const int t = static_cast<int>(row - b * n_token);
  const long long* idx = index + (b / index_div) * n_atom;
  const unsigned char* mk = mask + (b / index_div) * n_atom;
  const T* xb = x + b * n_atom * d;
  int a_begin = 0, a_end = n_atom;
  if (range != nullptr) {
    const int2 rg = range[(b / index_div) * n_token + t];
    a_begin = rg.x <= rg.y ? (rg.x & ~31) : 0;      // aligned to the 32-atom steps of the scan
    a_end = rg.x <= rg.y ? rg.y + 1 : 0;
  }
  for (int d0 = 0; d0 < d; d0 += kChunks * 32) {
    float acc[kChunks];
#pragma unroll
    for (int k = 0; k < kChunks; ++k) acc[k] = 0.f;
    int count = 0;
    for (int a0 = a_begin; a0 < a_end; a0 += 32) {
      const int a = a0 + lane;
      const bool hit = a < a_end && mk[a] != 0 && idx[a] == t;
      unsigned m = __ballot_sync(0xffffffffu, hit);
      count += __popc(m);
      while (m) {
        const int j = __ffs(m) - 1;
        m &= m - 1;
        const T* src = xb + static_cast<long long>(a0 + j) * d + d0;
#pragma unroll
        for (int k = 0; k < kChunks; ++k) {
          const int col = k * 32 + lane;
          if (d0 + col < d) {
            const float v = ld_f(src + col);
            acc[k] += relu ? fmaxf(v, 0.f) : v;
          }
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

KFB_API int kfb_tokens_to_atoms(const void* x, const long long* token_index, const void* addend, void* out, int batch,
                                int n_token, int n_atom, int d, int index_div, int x_dtype, int out_dtype, void* stream_) {
  KFB_CHECK_ARG(x && token_index && out, "tokens_to_atoms: null pointer");
  KFB_CHECK_ARG((x_dtype == KFB_BF16 || x_dtype == KFB_FP32) && (out_dtype == KFB_BF16 || out_dtype == KFB_FP32) &&
                    !(x_dtype == KFB_FP32 && out_dtype == KFB_BF16),
                "tokens_to_atoms: dtypes %d -> %d (bf16 -> bf16, bf16 -> fp32 or fp32 -> fp32)", x_dtype, out_dtype);
  KFB_CHECK_ARG(batch >= 1 && n_token >= 1 && n_atom >= 1 && d >= 1 && index_div >= 1 && batch % index_div == 0,
                "tokens_to_atoms: batch %d tokens %d atoms %d d %d index_div %d", batch, n_token, n_atom, d, index_div);
  cudaStream_t stream = as_stream(stream_);
  const long long rows = static_cast<long long>(batch) * n_atom;
  const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
  LaunchScope scope(stream, "tokens_to_atoms");
  using bf = __nv_bfloat16;
  if (x_dtype == KFB_BF16 && out_dtype == KFB_BF16)
    tokens_to_atoms_kernel<bf, bf><<<blocks, 256, 0, stream>>>(static_cast<const bf*>(x), token_index, static_cast<const bf*>(addend),
                                                               static_cast<bf*>(out), rows, n_atom, n_token, d, index_div);
  else if (x_dtype == KFB_BF16)
    tokens_to_atoms_kernel<bf, float><<<blocks, 256, 0, stream>>>(static_cast<const bf*>(x), token_index,
                                                                  static_cast<const float*>(addend), static_cast<float*>(out), rows,
                                                                  n_atom, n_token, d, index_div);
  else
    tokens_to_atoms_kernel<float, float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(x), token_index,
                                                                     static_cast<const float*>(addend), static_cast<float*>(out),
                                                                     rows, n_atom, n_token, d, index_div);
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

KFB_API size_t kfb_atoms_to_tokens_workspace_bytes(int batch, int n_token, int index_div) {
  return align_up(static_cast<size_t>(batch / (index_div > 0 ? index_div : 1)) * n_token * sizeof(int2), 256);
}

KFB_API int kfb_atoms_to_tokens(const void* x, const long long* token_index, const unsigned char* mask, void* out, void* workspace,
                                size_t workspace_bytes, int batch, int n_atom, int n_token, int d, int index_div, int relu,
                                int dtype, void* stream_) {
  KFB_CHECK_ARG(x && token_index && mask && out, "atoms_to_tokens: null pointer");
  KFB_CHECK_ARG(dtype == KFB_BF16 || dtype == KFB_FP32, "atoms_to_tokens: dtype %d (bf16 or fp32)", dtype);
  KFB_CHECK_ARG(batch >= 1 && n_token >= 1 && n_atom >= 1 && d >= 1 && index_div >= 1 && batch % index_div == 0,
                "atoms_to_tokens: batch %d tokens %d atoms %d d %d index_div %d", batch, n_token, n_atom, d, index_div);
  cudaStream_t stream = as_stream(stream_);
  const long long rows = static_cast<long long>(batch) * n_token;
  const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
  int2* range = nullptr;
  if (workspace != nullptr) {
    KFB_CHECK_ARG(workspace_bytes >= kfb_atoms_to_tokens_workspace_bytes(batch, n_token, index_div) &&
                      (reinterpret_cast<uintptr_t>(workspace) & 7) == 0,
                  "atoms_to_tokens: workspace too small or misaligned");
    range = static_cast<int2*>(workspace);
    const long long nr = static_cast<long long>(batch / index_div) * n_token, na = static_cast<long long>(batch / index_div) * n_atom;
    LaunchScope scope_r(stream, "atoms_to_tokens_ranges");
    token_range_init_kernel<<<static_cast<unsigned>((nr + 255) / 256), 256, 0, stream>>>(range, nr);
    token_range_kernel<<<static_cast<unsigned>((na + 255) / 256), 256, 0, stream>>>(token_index, mask, range, na, n_atom, n_token);
    KFB_CUDA(cudaGetLastError());
  }
  LaunchScope scope(stream, "atoms_to_tokens");
  if (dtype == KFB_BF16)
    atoms_to_tokens_kernel<__nv_bfloat16, 8><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), token_index, mask,
                                                                          static_cast<__nv_bfloat16*>(out), rows, n_atom, n_token, d,
                                                                          index_div, relu, range);
  else
    atoms_to_tokens_kernel<float, 8><<<blocks, 256, 0, stream>>>(static_cast<const float*>(x), token_index, mask,
                                                                  static_cast<float*>(out), rows, n_atom, n_token, d, index_div, relu,
                                                                  range);
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

KFB_API int kfb_coord_embed(const void* q, const float* r, const float* w, const unsigned char* mask, float* out, long long rows,
                            int c, int kc, int samples, int l, int q_dtype, void* stream_) {
  KFB_CHECK_ARG(q && r && w && out, "coord_embed: null pointer");
  KFB_CHECK_ARG(q_dtype == KFB_BF16 || q_dtype == KFB_FP32, "coord_embed: dtype %d (bf16 or fp32)", q_dtype);
  KFB_CHECK_ARG(rows >= 1 && c >= 1 && kc >= 1 && kc <= 8 && samples >= 1 && l >= 1 &&
                    rows % (static_cast<long long>(samples) * l) == 0,
                "coord_embed: rows %lld c %d coordinates %d samples %d l %d", rows, c, kc, samples, l);
  cudaStream_t stream = as_stream(stream_);
  const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
  LaunchScope scope(stream, "coord_embed");
  if (q_dtype == KFB_BF16)
    coord_embed_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(q), r, w, mask, out, rows, c, kc,
                                                                   samples, l);
  else
    coord_embed_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(q), r, w, mask, out, rows, c, kc, samples, l);
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

KFB_API int kfb_ln_project(const void* x, const float* ln_w, const float* ln_b, const float* w, const unsigned char* mask,
                           float* out, long long rows, int c, int n_out, float eps, int samples, int l, int dtype, void* stream_) {
  KFB_CHECK_ARG(x && w && out, "ln_project: null pointer");
  KFB_CHECK_ARG(dtype == KFB_BF16 || dtype == KFB_FP32, "ln_project: dtype %d (bf16 or fp32)", dtype);
  KFB_CHECK_ARG(rows >= 1 && c >= 1 && n_out >= 1 && n_out <= 8, "ln_project: rows %lld c %d outputs %d (at most 8)", rows, c, n_out);
  if (mask == nullptr) samples = l = 1;
  KFB_CHECK_ARG(samples >= 1 && l >= 1 && rows % (static_cast<long long>(samples) * l) == 0,
                "ln_project: rows %lld are not a multiple of samples %d x l %d", rows, samples, l);
  cudaStream_t stream = as_stream(stream_);
  const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
  LaunchScope scope(stream, "ln_project");
  if (dtype == KFB_BF16)
    ln_project_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), ln_w, ln_b, w, mask, out, rows,
                                                                  c, n_out, eps, samples, l);
  else
    ln_project_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(x), ln_w, ln_b, w, mask, out, rows, c, n_out, eps,
                                                         samples, l);
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

}  // extern "C"
