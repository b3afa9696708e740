// LayerNorm kernels.  Pure HBM traffic: every element is read once and written once,
// statistics are taken in fp32 with warp-shuffle reductions (two-pass: mean, then
// variance of the centred values, which is what torch's layer_norm computes).
#include "layernorm.cuh"

#include <type_traits>

namespace kfb {

template <typename T>
__device__ __forceinline__ float2 load2(const T* p);
template <>
__device__ __forceinline__ float2 load2<float>(const float* p) {
  return *reinterpret_cast<const float2*>(p);
}
template <>
__device__ __forceinline__ float2 load2<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <typename T>
__device__ __forceinline__ void store2(T* p, float a, float b);
template <>
__device__ __forceinline__ void store2<float>(float* p, float a, float b) {
  *reinterpret_cast<float2*>(p) = make_float2(a, b);
}
template <>
__device__ __forceinline__ void store2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per row; lane l holds channel pairs (l + 32 g) * 2, g < G.
template <typename TI, typename TO, int G, bool PERM>
__global__ void __launch_bounds__(256) layernorm_rows_kernel(const TI* __restrict__ x, TO* __restrict__ y,
                                                             const float* __restrict__ w, const float* __restrict__ b,
                                                             long long rows, int c, long long xs, long long ys, float eps,
                                                             RowPerm perm) {
  const int lane = threadIdx.x & 31;
  const long long warps_per_grid = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
       row += warps_per_grid) {
    const TI* xr = x + row * xs;
    float2 v[G];
    float s = 0.f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int ch = (lane + 32 * g) * 2;
      v[g] = ch < c ? load2<TI>(xr + ch) : make_float2(0.f, 0.f);
      s += v[g].x + v[g].y;
    }
    const float mean = warp_sum(s) / static_cast<float>(c);
    float q = 0.f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int ch = (lane + 32 * g) * 2;
      if (ch < c) {
        v[g].x -= mean;
        v[g].y -= mean;
        q += v[g].x * v[g].x + v[g].y * v[g].y;
      }
    }
    const float rstd = rsqrtf(warp_sum(q) / static_cast<float>(c) + eps);
    long long orow = row;
    if (PERM) {   // (i, q, j) -> (q, i, j): the send buffer of a shard transpose, one block per destination rank
      const long long i = row / perm.n;
      const int rest = static_cast<int>(row - i * perm.n);
      const int q = rest / perm.rows;
      orow = (static_cast<long long>(q) * perm.rows + i) * perm.rows + (rest - q * perm.rows);
    }
    TO* yr = y + orow * ys;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int ch = (lane + 32 * g) * 2;
      if (ch < c) {
        float a0 = v[g].x * rstd, a1 = v[g].y * rstd;
        if (w != nullptr) {
          const float2 ww = *reinterpret_cast<const float2*>(w + ch);
          a0 *= ww.x;
          a1 *= ww.y;
        }
        if (b != nullptr) {
          const float2 bb = *reinterpret_cast<const float2*>(b + ch);
          a0 += bb.x;
          a1 += bb.y;
        }
        store2<TO>(yr + ch, a0, a1);
      }
    }
  }
}

// The pair track's shape: 128 bf16 channels, contiguous rows.  A row is 256 bytes = 16 lanes x 16 bytes, so a warp takes two
// rows per step and two steps per iteration: four rows (1 KB) in flight per warp, 16-byte loads and stores, the statistics
// reduced over the 16 lanes of a row.  Same arithmetic as layernorm_rows_kernel (two passes, fp32).
__global__ void __launch_bounds__(256) layernorm_c128_bf16_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                                                  const float* __restrict__ w, const float* __restrict__ b,
                                                                  long long rows, float eps) {
  const int lane = threadIdx.x & 31;
  const int sub = lane & 15;                 // 16-byte chunk of the row
  const int half = lane >> 4;                // which of the warp's two rows
  float g[8], o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    g[i] = w != nullptr ? w[sub * 8 + i] : 1.0f;
    o[i] = b != nullptr ? b[sub * 8 + i] : 0.0f;
  }
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const long long warp_id = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  for (long long base = warp_id * 4; base < rows; base += warps * 4) {
    uint4 raw[2];
    bool live[2];
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const long long row = base + s * 2 + half;
      live[s] = row < rows;
      raw[s] = live[s] ? *reinterpret_cast<const uint4*>(x + row * 128 + sub * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const uint32_t wv[4] = {raw[s].x, raw[s].y, raw[s].z, raw[s].w};
      float v[8];
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(wv[i] << 16);
        v[2 * i + 1] = __uint_as_float(wv[i] & 0xffff0000u);
        sum += v[2 * i] + v[2 * i + 1];
      }
#pragma unroll
      for (int m = 8; m > 0; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
      const float mean = sum * (1.0f / 128.0f);
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i] -= mean;
        sq = fmaf(v[i], v[i], sq);
      }
#pragma unroll
      for (int m = 8; m > 0; m >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, m);
      const float rstd = rsqrtf(sq * (1.0f / 128.0f) + eps);
      uint4 out;
      uint32_t* ov = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 pr = __floats2bfloat162_rn(fmaf(v[2 * i] * rstd, g[2 * i], o[2 * i]),
                                                        fmaf(v[2 * i + 1] * rstd, g[2 * i + 1], o[2 * i + 1]));
        ov[i] = *reinterpret_cast<const uint32_t*>(&pr);
      }
      const long long row = base + s * 2 + half;
      if (live[s]) *reinterpret_cast<uint4*>(y + row * 128 + sub * 8) = out;
    }
  }
}

template <typename TI, typename TO, int G>
static int launch_rows(cudaStream_t stream, const void* x, void* y, const float* w, const float* b, long long rows, int c,
                       long long xs, long long ys, float eps, RowPerm perm) {
  const int warps = 8;
  long long blocks = (rows + warps - 1) / warps;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  LaunchScope scope(stream, "layernorm_rows");
  if (perm.rows) {
    if constexpr (std::is_same<TO, __nv_bfloat16>::value) {   // the exchange order is only ever written in bf16
      layernorm_rows_kernel<TI, TO, G, true><<<static_cast<unsigned>(blocks), warps * 32, 0, stream>>>(
          static_cast<const TI*>(x), static_cast<TO*>(y), w, b, rows, c, xs, ys, eps, perm);
    } else {
      set_error("layernorm: the exchange order is written in bf16 only");
      return KFB_ERR_UNSUPPORTED;
    }
  } else {
    layernorm_rows_kernel<TI, TO, G, false><<<static_cast<unsigned>(blocks), warps * 32, 0, stream>>>(
        static_cast<const TI*>(x), static_cast<TO*>(y), w, b, rows, c, xs, ys, eps, perm);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

template <typename TI, typename TO>
static int dispatch_g(cudaStream_t stream, const void* x, void* y, const float* w, const float* b, long long rows, int c,
                      long long xs, long long ys, float eps, RowPerm perm) {
  const int g = cdiv(c, 64);
  if (g <= 1) return launch_rows<TI, TO, 1>(stream, x, y, w, b, rows, c, xs, ys, eps, perm);
  if (g <= 2) return launch_rows<TI, TO, 2>(stream, x, y, w, b, rows, c, xs, ys, eps, perm);
  if (g <= 4) return launch_rows<TI, TO, 4>(stream, x, y, w, b, rows, c, xs, ys, eps, perm);
  if (g <= 6) return launch_rows<TI, TO, 6>(stream, x, y, w, b, rows, c, xs, ys, eps, perm);
  if (g <= 12) return launch_rows<TI, TO, 12>(stream, x, y, w, b, rows, c, xs, ys, eps, perm);
  if (g <= 16) return launch_rows<TI, TO, 16>(stream, x, y, w, b, rows, c, xs, ys, eps, perm);
  set_error("layernorm: channel count %d above 1024 is not supported", c);
  return KFB_ERR_UNSUPPORTED;
}

int launch_layernorm(cudaStream_t stream, const void* x, void* y, const float* w, const float* b, long long rows, int c,
                     long long xs, long long ys, float eps, int in_dtype, int out_dtype, RowPerm perm) {
  KFB_CHECK_ARG(rows >= 0 && c > 0 && c % 2 == 0, "layernorm: rows %lld, channels %d (must be even)", rows, c);
  KFB_CHECK_ARG(perm.rows == 0 || (perm.n % perm.rows == 0 && rows == static_cast<long long>(perm.rows) * perm.n),
                "layernorm: exchange order needs a (%d, %d) shard, got %lld rows", perm.rows, perm.n, rows);
  KFB_CHECK_ARG(xs % 2 == 0 && ys % 2 == 0, "layernorm: row strides must be even");
  if (rows == 0) return KFB_OK;
  if (in_dtype == KFB_BF16 && out_dtype == KFB_BF16 && c == 128 && xs == 128 && ys == 128 && perm.rows == 0 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0) {
    long long blocks = (rows + 31) / 32;      // 8 warps x 4 rows per iteration
    const long long cap = static_cast<long long>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    LaunchScope scope(stream, "layernorm_rows");
    layernorm_c128_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), w, b, rows, eps);
    KFB_CUDA(cudaGetLastError());
    return KFB_OK;
  }
  if (in_dtype == KFB_BF16 && out_dtype == KFB_BF16)
    return dispatch_g<__nv_bfloat16, __nv_bfloat16>(stream, x, y, w, b, rows, c, xs, ys, eps, perm);
  if (in_dtype == KFB_FP32 && out_dtype == KFB_BF16)
    return dispatch_g<float, __nv_bfloat16>(stream, x, y, w, b, rows, c, xs, ys, eps, perm);
  if (in_dtype == KFB_FP32 && out_dtype == KFB_FP32)
    return dispatch_g<float, float>(stream, x, y, w, b, rows, c, xs, ys, eps, perm);
  if (in_dtype == KFB_BF16 && out_dtype == KFB_FP32)
    return dispatch_g<__nv_bfloat16, float>(stream, x, y, w, b, rows, c, xs, ys, eps, perm);
  set_error("layernorm: bad dtype");
  return KFB_ERR_INVALID_ARGUMENT;
}

// ------------------------------------------------------------------------------------------------
// fp32-accurate mode: LayerNorm (or a plain copy) of fp32 rows, written as the bf16 triple split.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void split3_store(__nv_bfloat16* y6, int c, int ch, float v) {
  const __nv_bfloat16 x0 = __float2bfloat16_rn(v);
  const float r1 = v - __bfloat162float(x0);
  const __nv_bfloat16 x1 = __float2bfloat16_rn(r1);
  const __nv_bfloat16 x2 = __float2bfloat16_rn(r1 - __bfloat162float(x1));
  y6[ch] = x0; y6[c + ch] = x0; y6[2 * c + ch] = x1; y6[3 * c + ch] = x1; y6[4 * c + ch] = x0; y6[5 * c + ch] = x2;
}

__global__ void __launch_bounds__(256) layernorm_split_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y6,
                                                              const float* __restrict__ w, const float* __restrict__ b,
                                                              long long rows, int c, long long xs, float eps, int normalise) {
  const int lane = threadIdx.x & 31;
  const long long warps_per_grid = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
       row += warps_per_grid) {
    const float* xr = x + row * xs;
    float mean = 0.f, rstd = 1.f;
    if (normalise) {
      float s = 0.f;
      for (int ch = lane; ch < c; ch += 32) s += xr[ch];
      mean = warp_sum(s) / static_cast<float>(c);
      float q = 0.f;
      for (int ch = lane; ch < c; ch += 32) {
        const float d = xr[ch] - mean;
        q += d * d;
      }
      rstd = 1.0f / sqrtf(warp_sum(q) / static_cast<float>(c) + eps);
    }
    __nv_bfloat16* yr = y6 + row * 6 * c;
    for (int ch = lane; ch < c; ch += 32) {
      float v = (xr[ch] - mean) * rstd;
      if (w != nullptr) v *= w[ch];
      if (b != nullptr) v += b[ch];
      split3_store(yr, c, ch, v);
    }
  }
}

int launch_layernorm_split(cudaStream_t stream, const float* x, __nv_bfloat16* y6, const float* w, const float* b, long long rows,
                           int c, long long xs, float eps, int normalise) {
  KFB_CHECK_ARG(rows >= 0 && c > 0, "layernorm_split: rows %lld, channels %d", rows, c);
  if (rows == 0) return KFB_OK;
  const int warps = 8;
  long long blocks = (rows + warps - 1) / warps;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  LaunchScope scope(stream, "layernorm_split");
  layernorm_split_kernel<<<static_cast<unsigned>(blocks), warps * 32, 0, stream>>>(x, y6, w, b, rows, c, xs, eps, normalise);
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

// Channel-major fp32 in, position-major triple split out (fp32-accurate mode): fp32 slab, one thread per position.
__global__ void __launch_bounds__(128) layernorm_cm_split_kernel(const float* __restrict__ t, __nv_bfloat16* __restrict__ y6,
                                                                 const float* __restrict__ w, const float* __restrict__ b,
                                                                 long long npos, int c, long long chan_stride,
                                                                 long long batch_stride, float eps, int blocks_per_batch) {
  extern __shared__ __align__(16) unsigned char slab_raw_f[];
  float* slab = reinterpret_cast<float*>(slab_raw_f);  // [c][128]
  const int batch = blockIdx.x / blocks_per_batch;
  const long long p0 = static_cast<long long>(blockIdx.x % blocks_per_batch) * 128;
  const float* tb = t + batch * batch_stride + p0;
  for (int idx = threadIdx.x; idx < c * 128; idx += 128) {
    const int ch = idx >> 7, pp = idx & 127;
    slab[idx] = (p0 + pp < npos) ? tb[ch * chan_stride + pp] : 0.f;
  }
  __syncthreads();
  const long long p = p0 + threadIdx.x;
  if (p >= npos) return;
  const float* col = slab + threadIdx.x;
  float s = 0.f;
  for (int ch = 0; ch < c; ++ch) s += col[ch * 128];
  const float mean = s / static_cast<float>(c);
  float q = 0.f;
  for (int ch = 0; ch < c; ++ch) {
    const float d = col[ch * 128] - mean;
    q += d * d;
  }
  const float rstd = 1.0f / sqrtf(q / static_cast<float>(c) + eps);
  __nv_bfloat16* yr = y6 + (static_cast<long long>(batch) * npos + p) * 6 * c;
  for (int ch = 0; ch < c; ++ch) {
    float v = (col[ch * 128] - mean) * rstd;
    if (w != nullptr) v *= w[ch];
    if (b != nullptr) v += b[ch];
    split3_store(yr, c, ch, v);
  }
}

// ------------------------------------------------------------------------------------------------
// Adaptive LayerNorm (AdaLN): one warp per row, same register layout as layernorm_rows_kernel.
// ------------------------------------------------------------------------------------------------
template <typename TI, typename TO, typename TG, int G>
__global__ void __launch_bounds__(256) adaln_rows_kernel(const TI* __restrict__ a, TO* __restrict__ y,
                                                         const TG* __restrict__ gv, long long gv_ld, long long rows, int c,
                                                         int samples, int l, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warps_per_grid = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
       row += warps_per_grid) {
    const TI* xr = a + row * c;
    const long long srow = (row / (static_cast<long long>(samples) * l)) * l + row % l;
    const TG* gr = gv + srow * gv_ld;
    float2 v[G], gate[G], shift[G];
    float s = 0.f;
    // the gate / shift rows do not depend on the statistics: their loads are issued together with the row's own
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int ch = (lane + 32 * g) * 2;
      v[g] = ch < c ? load2<TI>(xr + ch) : make_float2(0.f, 0.f);
      gate[g] = ch < c ? load2<TG>(gr + ch) : make_float2(0.f, 0.f);
      shift[g] = ch < c ? load2<TG>(gr + c + ch) : make_float2(0.f, 0.f);
      s += v[g].x + v[g].y;
    }
    const float mean = warp_sum(s) / static_cast<float>(c);
    float q = 0.f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int ch = (lane + 32 * g) * 2;
      if (ch < c) {
        v[g].x -= mean;
        v[g].y -= mean;
        q += v[g].x * v[g].x + v[g].y * v[g].y;
      }
    }
    const float rstd = rsqrtf(warp_sum(q) / static_cast<float>(c) + eps);
    TO* yr = y + row * c;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int ch = (lane + 32 * g) * 2;
      if (ch < c) {
        const float s0 = 1.f / (1.f + __expf(-gate[g].x)), s1 = 1.f / (1.f + __expf(-gate[g].y));
        store2<TO>(yr + ch, s0 * (v[g].x * rstd) + shift[g].x, s1 * (v[g].y * rstd) + shift[g].y);
      }
    }
  }
}

// bf16 rows of 256 * CH channels (the token transformer's 768, 1024): 16-byte accesses, CH per lane for each of the row,
// its gate row and its shift row (3 * CH loads in flight per lane instead of 36 four-byte ones at c = 768); the sigmoid as
// 0.5 + 0.5 tanh(g / 2) on the MUFU (one op instead of an exponential and a reciprocal; relative error 5e-4, below the
// bf16 rounding of the result).  LANES = 32: one row per warp; LANES = 16 (CH = 1, c = 128: the atom transformer):
// two rows per warp.
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  unpack8(*reinterpret_cast<const uint4*>(p), f);
}
__device__ __forceinline__ void load8(const float* p, float (&f)[8]) {
  const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 4);
  f[0] = lo.x; f[1] = lo.y; f[2] = lo.z; f[3] = lo.w; f[4] = hi.x; f[5] = hi.y; f[6] = hi.z; f[7] = hi.w;
}
template <typename TI, int CH, int LANES>
__global__ void __launch_bounds__(256) adaln_vec_kernel(const TI* __restrict__ a, __nv_bfloat16* __restrict__ y,
                                                        const __nv_bfloat16* __restrict__ gv, long long gv_ld, long long rows,
                                                        int samples, int l, float eps) {
  constexpr int c = 8 * LANES * CH;
  constexpr int kRowsPerWarp = 32 / LANES;
  const int lane = threadIdx.x & 31;
  const int sub = lane % LANES;
  const long long warps_per_grid = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long base = (static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kRowsPerWarp; base < rows;
       base += warps_per_grid * kRowsPerWarp) {
    const long long row = base + lane / LANES;
    const bool live = row < rows;
    const long long rr = live ? row : 0;
    const long long srow = (rr / (static_cast<long long>(samples) * l)) * l + rr % l;
    const TI* xr = a + rr * c;
    const __nv_bfloat16* gr = gv + srow * gv_ld;
    uint4 gt[CH], sh[CH];
    float v[CH][8];
#pragma unroll
    for (int k = 0; k < CH; ++k) {
      const int ch = (sub + LANES * k) * 8;
      load8(xr + ch, v[k]);
      gt[k] = *reinterpret_cast<const uint4*>(gr + ch);
      sh[k] = *reinterpret_cast<const uint4*>(gr + c + ch);
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < CH; ++k)
#pragma unroll
      for (int i = 0; i < 8; ++i) s += v[k][i];
#pragma unroll
    for (int m = LANES / 2; m > 0; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
    const float mean = s * (1.0f / c);
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < CH; ++k)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[k][i] -= mean;
        q = fmaf(v[k][i], v[k][i], q);
      }
#pragma unroll
    for (int m = LANES / 2; m > 0; m >>= 1) q += __shfl_xor_sync(0xffffffffu, q, m);
    const float rstd = rsqrtf(q * (1.0f / c) + eps);
    if (live) {
      __nv_bfloat16* yr = y + row * c;
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        float g[8], t[8];
        unpack8(gt[k], g);
        unpack8(sh[k], t);
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float t0, t1;
          asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(0.5f * g[2 * i]));
          asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(0.5f * g[2 * i + 1]));
          const __nv_bfloat162 pr = __floats2bfloat162_rn(fmaf(fmaf(t0, 0.5f, 0.5f), v[k][2 * i] * rstd, t[2 * i]),
                                                          fmaf(fmaf(t1, 0.5f, 0.5f), v[k][2 * i + 1] * rstd, t[2 * i + 1]));
          o[i] = *reinterpret_cast<const uint32_t*>(&pr);
        }
        *reinterpret_cast<uint4*>(yr + (sub + LANES * k) * 8) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

template <typename TI, int CH, int LANES>
static int launch_adaln_vec(cudaStream_t stream, const void* a, void* y, const void* gv, long long gv_ld, long long rows, int samples,
                            int l, float eps) {
  const long long rows_per_block = 8 * (32 / LANES);
  long long blocks = (rows + rows_per_block - 1) / rows_per_block;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  LaunchScope scope(stream, "adaln_rows");
  adaln_vec_kernel<TI, CH, LANES><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const TI*>(a), static_cast<__nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(gv), gv_ld, rows,
      samples, l, eps);
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

template <typename TI, typename TO, typename TG>
static int adaln_dispatch(cudaStream_t stream, const void* a, void* y, const void* gv_, long long gv_ld, long long rows, int c,
                          int samples, int l, float eps) {
  const TG* gv = static_cast<const TG*>(gv_);
  const int warps = 8;
  long long blocks = (rows + warps - 1) / warps;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  const int g = cdiv(c, 64);
  LaunchScope scope(stream, "adaln_rows");
#define KFB_ADALN(GG)                                                                                          \
  adaln_rows_kernel<TI, TO, TG, GG><<<static_cast<unsigned>(blocks), warps * 32, 0, stream>>>(                  \
      static_cast<const TI*>(a), static_cast<TO*>(y), gv, gv_ld, rows, c, samples, l, eps)
  if (g <= 2) KFB_ADALN(2);
  else if (g <= 6) KFB_ADALN(6);
  else if (g <= 12) KFB_ADALN(12);
  else if (g <= 16) KFB_ADALN(16);
  else {
    set_error("adaln: channel count %d above 1024 is not supported", c);
    return KFB_ERR_UNSUPPORTED;
  }
#undef KFB_ADALN
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

int launch_adaln(cudaStream_t stream, const void* a, void* y, const void* gv, long long rows, int c, int samples,
                 int l, float eps, int in_dtype, int out_dtype, long long gv_ld) {
  if (gv_ld <= 0) gv_ld = 2ll * c;
  KFB_CHECK_ARG(gv_ld >= 2ll * c && gv_ld % 2 == 0 && (reinterpret_cast<uintptr_t>(gv) & 7) == 0,
                "adaln: gate/shift row stride %lld (at least 2c, even) or misaligned pointer", gv_ld);
  KFB_CHECK_ARG(rows >= 0 && c > 0 && c % 2 == 0 && samples >= 1 && l >= 1, "adaln: rows %lld c %d samples %d l %d", rows, c,
                samples, l);
  KFB_CHECK_ARG(rows % (static_cast<long long>(samples) * l) == 0, "adaln: rows %lld is not a multiple of samples*l", rows);
  if (rows == 0) return KFB_OK;
  if ((in_dtype == KFB_BF16 || in_dtype == KFB_FP32) && out_dtype == KFB_BF16 && gv_ld % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(gv)) & 15) == 0) {
#define KFB_ADALN_VEC(CH, LANES)                                                                                          \
  return in_dtype == KFB_BF16 ? launch_adaln_vec<__nv_bfloat16, CH, LANES>(stream, a, y, gv, gv_ld, rows, samples, l, eps) \
                              : launch_adaln_vec<float, CH, LANES>(stream, a, y, gv, gv_ld, rows, samples, l, eps)
    switch (c) {
      case 128: KFB_ADALN_VEC(1, 16);
      case 256: KFB_ADALN_VEC(1, 32);
      case 512: KFB_ADALN_VEC(2, 32);
      case 768: KFB_ADALN_VEC(3, 32);
      case 1024: KFB_ADALN_VEC(4, 32);
      default: break;
    }
#undef KFB_ADALN_VEC
  }
  if (in_dtype == KFB_BF16 && out_dtype == KFB_BF16)
    return adaln_dispatch<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(stream, a, y, gv, gv_ld, rows, c, samples, l, eps);
  if (in_dtype == KFB_FP32 && out_dtype == KFB_BF16)
    return adaln_dispatch<float, __nv_bfloat16, __nv_bfloat16>(stream, a, y, gv, gv_ld, rows, c, samples, l, eps);
  if (in_dtype == KFB_FP32_PRECISE && out_dtype == KFB_FP32)  // everything fp32, gate / shift rows included
    return adaln_dispatch<float, float, float>(stream, a, y, gv, gv_ld, rows, c, samples, l, eps);
  set_error("adaln: unsupported dtype combination");
  return KFB_ERR_INVALID_ARGUMENT;
}

// ------------------------------------------------------------------------------------------------
// Channel-major in, position-major out.  A block of 128 threads stages a [c][128 positions] slab in shared
// memory as bf16 (each warp copies whole channel rows: 256 contiguous bytes per row), then every thread
// owns ONE position: it walks down its column of the slab (neighbouring lanes read neighbouring 2-byte
// cells, so the column walk is bank-conflict free), takes mean and variance in two passes and writes its
// normalised row of c channels with 16-byte stores.
// ------------------------------------------------------------------------------------------------
static constexpr int kCmPos = 128;

__device__ __forceinline__ float cm_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float cm_to_float(float v) { return v; }
__device__ __forceinline__ uint32_t cm_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <typename TI>
__global__ void __launch_bounds__(kCmPos) layernorm_cm_kernel(const TI* __restrict__ t, __nv_bfloat16* __restrict__ y,
                                                              const float* __restrict__ w, const float* __restrict__ b,
                                                              long long npos, int c, long long chan_stride,
                                                              long long batch_stride, float eps, int blocks_per_batch) {
  extern __shared__ __align__(16) unsigned char slab_raw[];
  __nv_bfloat16* slab = reinterpret_cast<__nv_bfloat16*>(slab_raw);  // [c][128]
  const int batch = blockIdx.x / blocks_per_batch;
  const long long p0 = static_cast<long long>(blockIdx.x % blocks_per_batch) * kCmPos;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TI* tb = t + batch * batch_stride + p0;
  const bool full = (p0 + kCmPos <= npos) && ((chan_stride & 3) == 0) && ((reinterpret_cast<uintptr_t>(tb) & 7) == 0);
  for (int ch = warp; ch < c; ch += kCmPos / 32) {
    const TI* src = tb + ch * chan_stride + lane * 4;
    __nv_bfloat16* dst = slab + ch * kCmPos + lane * 4;
    if (full && sizeof(TI) == 2) {
      *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(src);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        dst[i] = (p0 + lane * 4 + i < npos) ? __float2bfloat16_rn(cm_to_float(src[i])) : __float2bfloat16_rn(0.f);
    }
  }
  __syncthreads();
  const long long p = p0 + threadIdx.x;
  if (p >= npos) return;
  const __nv_bfloat16* col = slab + threadIdx.x;
  // mean and variance in one walk down the column, as sums of (x - x0) and (x - x0)^2 with x0 the first channel:
  // the shift keeps the subtraction of the squared mean harmless
  const float x0 = __bfloat162float(col[0]);
  float s = 0.f, q2 = 0.f;
#pragma unroll 8
  for (int ch = 0; ch < c; ++ch) {
    const float d = __bfloat162float(col[ch * kCmPos]) - x0;
    s += d;
    q2 = fmaf(d, d, q2);
  }
  const float ms = s / static_cast<float>(c);
  const float mean = x0 + ms;
  const float q = fmaxf(q2 - s * ms, 0.f);
  const float rstd = rsqrtf(q / static_cast<float>(c) + eps);
  __nv_bfloat16* yr = y + (static_cast<long long>(batch) * npos + p) * c;
  if ((c & 15) == 0 && (reinterpret_cast<uintptr_t>(yr) & 31) == 0) {
    for (int ch = 0; ch < c; ch += 16) {   // 32-byte stores: one full sector per instruction
      uint32_t o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float a0 = (__bfloat162float(col[(ch + 2 * i) * kCmPos]) - mean) * rstd;
        float a1 = (__bfloat162float(col[(ch + 2 * i + 1) * kCmPos]) - mean) * rstd;
        if (w != nullptr) { a0 *= w[ch + 2 * i]; a1 *= w[ch + 2 * i + 1]; }
        if (b != nullptr) { a0 += b[ch + 2 * i]; a1 += b[ch + 2 * i + 1]; }
        o[i] = cm_pack(a0, a1);
      }
      asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(yr + ch), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                   "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                   : "memory");
    }
    return;
  }
  for (int ch = 0; ch < c; ch += 8) {
    float a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a[i] = (__bfloat162float(col[(ch + i) * kCmPos]) - mean) * rstd;
      if (w != nullptr) a[i] *= w[ch + i];
      if (b != nullptr) a[i] += b[ch + i];
    }
    *reinterpret_cast<uint4*>(yr + ch) = make_uint4(cm_pack(a[0], a[1]), cm_pack(a[2], a[3]), cm_pack(a[4], a[5]), cm_pack(a[6], a[7]));
  }
}

// ------------------------------------------------------------------------------------------------
// LayerNorm folded into the GEMM that follows it.  For rows x (c channels) and a projection W,
//   LN(x) W^T = rstd * (x W'^T - mean * s1) + s0,   W' = gamma * W,  s1[n] = sum_k W'[n][k],  s0[n] = sum_k beta[k] W[n][k],
// so the GEMM can read the raw rows (here: channel-major, as the triangle contraction leaves them) and the epilogue
// applies the per-row (mean, rstd) and the per-column s1, s0.  Two small kernels prepare those.
// ------------------------------------------------------------------------------------------------
// (mean, rstd) over the channels of every position of a channel-major tensor t[c][npos]; two positions per thread
__global__ void __launch_bounds__(256) cm_stats_kernel(const __nv_bfloat16* __restrict__ t, float2* __restrict__ stats,
                                                       long long npos, int c, long long chan_stride, float eps) {
  const long long p2 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 2;
  if (p2 >= npos) return;
  const bool pair = p2 + 1 < npos;
  float s0 = 0.f, s1 = 0.f, q0 = 0.f, q1 = 0.f;
  // shifted sums (by the first channel's value) keep E[x^2] - E[x]^2 harmless
  float x00, x01;
  {
    const __nv_bfloat16* src = t + p2;
    x00 = __bfloat162float(src[0]);
    x01 = pair ? __bfloat162float(src[1]) : 0.f;
  }
#pragma unroll 8
  for (int ch = 0; ch < c; ++ch) {
    const __nv_bfloat16* src = t + ch * chan_stride + p2;
    float a, b2;
    if (pair) {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(src);
      a = __uint_as_float(w << 16);
      b2 = __uint_as_float(w & 0xffff0000u);
    } else {
      a = __bfloat162float(src[0]);
      b2 = 0.f;
    }
    const float d0 = a - x00, d1 = b2 - x01;
    s0 += d0; q0 = fmaf(d0, d0, q0);
    s1 += d1; q1 = fmaf(d1, d1, q1);
  }
  const float inv_c = 1.0f / static_cast<float>(c);
  const float m0 = s0 * inv_c, m1 = s1 * inv_c;
  stats[p2] = make_float2(x00 + m0, rsqrtf(fmaxf(q0 - s0 * m0, 0.f) * inv_c + eps));
  if (pair) stats[p2 + 1] = make_float2(x01 + m1, rsqrtf(fmaxf(q1 - s1 * m1, 0.f) * inv_c + eps));
}

// The same with four positions per thread (8-byte loads): half as many CTAs, all resident at once for a 768 x 768 pair
// tensor, and twice the bytes in flight per thread.  npos and the channel stride multiples of 4, t 8-byte aligned.
__global__ void __launch_bounds__(128) cm_stats4_kernel(const __nv_bfloat16* __restrict__ t, float2* __restrict__ stats,
                                                        long long npos, int c, long long chan_stride, float eps) {
  const long long p4 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (p4 >= npos) return;
  float s[4] = {0.f, 0.f, 0.f, 0.f}, q[4] = {0.f, 0.f, 0.f, 0.f}, x0[4];
  {
    const uint2 w = *reinterpret_cast<const uint2*>(t + p4);
    x0[0] = __uint_as_float(w.x << 16);
    x0[1] = __uint_as_float(w.x & 0xffff0000u);
    x0[2] = __uint_as_float(w.y << 16);
    x0[3] = __uint_as_float(w.y & 0xffff0000u);
  }
#pragma unroll 8
  for (int ch = 0; ch < c; ++ch) {
    const uint2 w = *reinterpret_cast<const uint2*>(t + ch * chan_stride + p4);
    const float v[4] = {__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u), __uint_as_float(w.y << 16),
                        __uint_as_float(w.y & 0xffff0000u)};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float d = v[i] - x0[i];
      s[i] += d;
      q[i] = fmaf(d, d, q[i]);
    }
  }
  const float inv_c = 1.0f / static_cast<float>(c);
  float4 o[2];
  float* of = reinterpret_cast<float*>(o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float m = s[i] * inv_c;
    of[2 * i] = x0[i] + m;
    of[2 * i + 1] = rsqrtf(fmaxf(q[i] - s[i] * m, 0.f) * inv_c + eps);
  }
  float4* dst = reinterpret_cast<float4*>(stats + p4);
  dst[0] = o[0];
  dst[1] = o[1];
}

int launch_cm_stats(cudaStream_t stream, const __nv_bfloat16* t, float2* stats, long long npos, int c, long long chan_stride,
                    float eps) {
  KFB_CHECK_ARG(npos > 0 && npos % 2 == 0 && c > 0 && chan_stride % 2 == 0 && (reinterpret_cast<uintptr_t>(t) & 3) == 0,
                "cm_stats: npos %lld (even), c %d, channel stride %lld (even)", npos, c, chan_stride);
  LaunchScope scope(stream, "layernorm_cm_stats");
  if (npos % 4 == 0 && chan_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(t) & 7) == 0 &&
      (reinterpret_cast<uintptr_t>(stats) & 15) == 0) {
    const long long threads4 = npos / 4;
    cm_stats4_kernel<<<static_cast<unsigned>((threads4 + 127) / 128), 128, 0, stream>>>(t, stats, npos, c, chan_stride, eps);
    KFB_CUDA(cudaGetLastError());
    return KFB_OK;
  }
  const long long threads = npos / 2;
  cm_stats_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(t, stats, npos, c, chan_stride, eps);
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

// W'[n][k] = bf16(gamma[k] W[n][k]); s1[n] = sum_k W'[n][k] (of the rounded values); s0[n] = sum_k beta[k] W[n][k]
__global__ void __launch_bounds__(128) ln_fold_weights_kernel(const __nv_bfloat16* __restrict__ w, const float* __restrict__ gamma,
                                                              const float* __restrict__ beta, __nv_bfloat16* __restrict__ wf,
                                                              float* __restrict__ s1, float* __restrict__ s0, int k) {
  const int n = blockIdx.x;
  float a1 = 0.f, a0 = 0.f;
  for (int i = threadIdx.x; i < k; i += blockDim.x) {
    const float wv = __bfloat162float(w[static_cast<long long>(n) * k + i]);
    const __nv_bfloat16 f = __float2bfloat16_rn(wv * (gamma != nullptr ? gamma[i] : 1.0f));
    wf[static_cast<long long>(n) * k + i] = f;
    a1 += __bfloat162float(f);
    a0 += (beta != nullptr ? beta[i] : 0.0f) * wv;
  }
  __shared__ float r1[4], r0[4];
  a1 = warp_sum(a1);
  a0 = warp_sum(a0);
  if ((threadIdx.x & 31) == 0) { r1[threadIdx.x >> 5] = a1; r0[threadIdx.x >> 5] = a0; }
  __syncthreads();
  if (threadIdx.x == 0) {
    s1[n] = (r1[0] + r1[1]) + (r1[2] + r1[3]);
    s0[n] = (r0[0] + r0[1]) + (r0[2] + r0[3]);
  }
}

int launch_ln_fold_weights(cudaStream_t stream, const __nv_bfloat16* w, const float* gamma, const float* beta, __nv_bfloat16* wf,
                           float* s1, float* s0, int n, int k) {
  KFB_CHECK_ARG(n > 0 && k > 0, "ln_fold_weights: n %d k %d", n, k);
  LaunchScope scope(stream, "layernorm_fold_weights");
  ln_fold_weights_kernel<<<n, 128, 0, stream>>>(w, gamma, beta, wf, s1, s0, k);
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_float(float v) { return v; }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }

// LayerNorm over a few channels followed by a projection to `nh` head values, one thread per position: the pair
// bias of the atom windows (16 channels in, heads x layers out).  x [npos][C]; w [nh][C]; y [nh][npos] (head-major,
// positions contiguous).  bf16 mode rounds the normalised value to bf16 as the reference's LayerNorm does and
// accumulates in fp32; fp32 mode keeps everything in fp32.
template <int C, typename T>
__global__ void __launch_bounds__(256) window_bias_kernel(const T* __restrict__ x, const float* __restrict__ ln_w,
                                                          const float* __restrict__ ln_b, const T* __restrict__ w,
                                                          T* __restrict__ y, long long npos, int nh, float eps, int normalise) {
  extern __shared__ float s_w[];  // [nh][C] fp32, then gamma[C], beta[C]
  float* s_g = s_w + nh * C;
  float* s_b = s_g + C;
  for (int i = threadIdx.x; i < nh * C; i += blockDim.x) s_w[i] = to_float(w[i]);
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    s_g[i] = ln_w != nullptr ? ln_w[i] : 1.0f;
    s_b[i] = ln_b != nullptr ? ln_b[i] : 0.0f;
  }
  __syncthreads();
  const long long pos = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (pos >= npos) return;
  float v[C];
  const T* xr = x + pos * C;
  constexpr int kVec = 16 / sizeof(T);
#pragma unroll
  for (int i = 0; i < C; i += kVec) {
    const uint4 raw = *reinterpret_cast<const uint4*>(xr + i);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < kVec; ++j) v[i + j] = to_float(e[j]);
  }
  if (normalise) {
    float mean = 0.f;
#pragma unroll
    for (int i = 0; i < C; ++i) mean += v[i];
    mean *= 1.0f / C;
    float var = 0.f;
#pragma unroll
    for (int i = 0; i < C; ++i) var += (v[i] - mean) * (v[i] - mean);
    const float rstd = rsqrtf(var * (1.0f / C) + eps);
#pragma unroll
    for (int i = 0; i < C; ++i) v[i] = to_float(from_float<T>((v[i] - mean) * rstd * s_g[i] + s_b[i]));
  }
  for (int h = 0; h < nh; ++h) {
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < C; ++i) acc = fmaf(v[i], s_w[h * C + i], acc);
    y[static_cast<long long>(h) * npos + pos] = from_float<T>(acc);
  }
}

template <int C>
static int launch_window_bias_c(cudaStream_t stream, const void* x, const float* ln_w, const float* ln_b, const void* w, void* y,
                                long long npos, int nh, float eps, int normalise, int dtype) {
  const size_t smem = (static_cast<size_t>(nh) * C + 2 * C) * sizeof(float);
  const unsigned blocks = static_cast<unsigned>((npos + 255) / 256);
  LaunchScope scope(stream, "window_bias");
  if (dtype == KFB_BF16)
    window_bias_kernel<C, __nv_bfloat16><<<blocks, 256, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(x), ln_w, ln_b, static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y),
        npos, nh, eps, normalise);
  else
    window_bias_kernel<C, float><<<blocks, 256, smem, stream>>>(static_cast<const float*>(x), ln_w, ln_b,
                                                                static_cast<const float*>(w), static_cast<float*>(y), npos, nh, eps,
                                                                normalise);
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

int launch_window_bias(cudaStream_t stream, const void* x, const float* ln_w, const float* ln_b, const void* w, void* y,
                       long long npos, int c, int nh, float eps, int normalise, int dtype) {
  KFB_CHECK_ARG(dtype == KFB_BF16 || dtype == KFB_FP32, "window_bias: dtype %d (bf16 or fp32)", dtype);
  KFB_CHECK_ARG(nh >= 1 && nh * c <= 8192, "window_bias: %d heads x %d channels exceed the shared-memory weight table", nh, c);
  KFB_CHECK_ARG(npos < (1ll << 31) * 256, "window_bias: too many positions");
  if (npos == 0) return KFB_OK;
  switch (c) {
    case 16: return launch_window_bias_c<16>(stream, x, ln_w, ln_b, w, y, npos, nh, eps, normalise, dtype);
    case 32: return launch_window_bias_c<32>(stream, x, ln_w, ln_b, w, y, npos, nh, eps, normalise, dtype);
    case 64: return launch_window_bias_c<64>(stream, x, ln_w, ln_b, w, y, npos, nh, eps, normalise, dtype);
    default:
      set_error("window_bias: %d channels not supported (16, 32 or 64)", c);
      return KFB_ERR_UNSUPPORTED;
  }
}

int launch_layernorm_cm(cudaStream_t stream, const void* t, __nv_bfloat16* y, const float* w, const float* b, int batch,
                        long long npos, int c, long long chan_stride, long long batch_stride, float eps, int in_dtype,
                        int split_out) {
  KFB_CHECK_ARG(c > 0 && c % 8 == 0 && c <= 512, "layernorm_cm: channels %d (multiple of 8, at most 512)", c);
  if (split_out) {
    KFB_CHECK_ARG(in_dtype == KFB_FP32 && c <= 256, "layernorm_cm: the split output takes fp32 input and at most 256 channels");
    if (npos == 0 || batch == 0) return KFB_OK;
    const int bpb = static_cast<int>((npos + 127) / 128);
    const size_t smem = static_cast<size_t>(c) * 128 * sizeof(float);
    if (smem > 48 * 1024)
      KFB_CUDA(cudaFuncSetAttribute(layernorm_cm_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LaunchScope scope(stream, "layernorm_cm_split");
    layernorm_cm_split_kernel<<<bpb * batch, 128, smem, stream>>>(static_cast<const float*>(t), y, w, b, npos, c, chan_stride,
                                                                 batch_stride, eps, bpb);
    KFB_CUDA(cudaGetLastError());
    return KFB_OK;
  }
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(y) & 15) == 0, "layernorm_cm: output must be 16-byte aligned");
  if (npos == 0 || batch == 0) return KFB_OK;
  const int bpb = static_cast<int>((npos + kCmPos - 1) / kCmPos);
  const size_t smem = static_cast<size_t>(c) * kCmPos * sizeof(__nv_bfloat16);
  LaunchScope scope(stream, "layernorm_cm");
  if (in_dtype == KFB_BF16) {
    if (smem > 48 * 1024)
      KFB_CUDA(cudaFuncSetAttribute(layernorm_cm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    layernorm_cm_kernel<__nv_bfloat16><<<bpb * batch, kCmPos, smem, stream>>>(static_cast<const __nv_bfloat16*>(t), y, w, b, npos,
                                                                           c, chan_stride, batch_stride, eps, bpb);
  } else {
    if (smem > 48 * 1024)
      KFB_CUDA(cudaFuncSetAttribute(layernorm_cm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    layernorm_cm_kernel<float><<<bpb * batch, kCmPos, smem, stream>>>(static_cast<const float*>(t), y, w, b, npos, c, chan_stride,
                                                                   batch_stride, eps, bpb);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

}  // namespace kfb
