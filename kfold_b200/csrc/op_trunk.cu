// Callers of the pair stacks in K-Fold's trunk (model/model.py:477-534).
//   kfb_parcae_fwd        z <- a * z + Linear_b(LayerNorm(u))       the recurrence between the recycling iterations
//   kfb_lm_pair_features  [xi * xj | xi - xj] for every token pair    the outer-product features of LMToPair
//   kfb_gelu              erf GELU, element-wise                      the activation inside LMToPair's MLP
// of the diffusion module's pair conditioning (model/layers/folding/diffusion.py:45-94):
//   kfb_concat_layernorm  LayerNorm([z | relative-position features])  one pass, written K-padded for the float32 Linear
//   kfb_relpos_concat_layernorm  the same with the features computed from the token attributes (never stored)
// and of the confidence head (model/modules/confidence_head.py:306-470):
//   kfb_pair_outer_add       z + Linear_1(s)[j] + Linear_2(s)[i]       the single representation added along both token axes
//   kfb_distogram_embed_add  z + Linear(one_hot(distance bin))         the predicted structure's distogram, embedded
#include "ops_common.cuh"

using namespace kfb;

namespace {

template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// out[(i, j), 0:d] = xi[i] * xj[j], out[(i, j), d:2d] = xi[i] - xj[j] with [xi | xj] = x[token, 0:2d]; bf16 out.
// One block per (batch, i); thread t walks (j, channel) pairs with the channel fastest: coalesced 2-byte stores.
template <typename T>
__global__ void __launch_bounds__(256) lm_pair_features_kernel(const T* __restrict__ x, __nv_bfloat16* __restrict__ out, int n, int d) {
  const int bi = blockIdx.x;            // batch * n + i
  const int b = bi / n;
  const T* xi = x + static_cast<long long>(bi) * 2 * d;
  const T* xb = x + static_cast<long long>(b) * n * 2 * d;
  __nv_bfloat16* o = out + static_cast<long long>(bi) * n * 2 * d;
  const int total = n * d;
  for (int e = threadIdx.x; e < total; e += 256) {
    const int j = e / d, ch = e - j * d;
    const float a = ldf(xi + ch), c = ldf(xb + static_cast<long long>(j) * 2 * d + d + ch);
    o[static_cast<long long>(j) * 2 * d + ch] = __float2bfloat16_rn(a * c);
    o[static_cast<long long>(j) * 2 * d + d + ch] = __float2bfloat16_rn(a - c);
  }
}

// y[row, 0:c1+c2] = LayerNorm([z[row, 0:c1] | rel[row, 0:c2]]) * w (+ b), y[row, c1+c2 : k_pad] = 0, float32 out.  One warp per
// row, the row held in registers (up to 32 * kMaxPerLane channels), mean and variance in two register passes.
constexpr int kCatPerLane = 16;

// The second part of the concatenated row, stored ...
template <typename TR>
struct StoredFeatures {
  const TR* rel;
  int c2;
  struct Row {
    const TR* p;
    __device__ __forceinline__ float at(int k) const { return ldf(p + k); }
  };
  __device__ __forceinline__ Row row(long long r) const { return Row{rel + r * c2}; }
};
// ... or the relative-position encoding computed from the token attributes (model/layers/folding/embeddings.py:58-130):
// [one_hot(residue offset, 2 r_max + 2) | one_hot(token offset, 2 r_max + 2) | same entity | one_hot(chain offset, 2 s_max + 2)],
// offsets clipped to [0, 2 max] and moved to the last bin when the tokens are not comparable (other chain; other chain or
// residue; other entity).
struct RelPosFeatures {
  const long long *asym, *residue, *entity, *token, *sym;   // [batch][n] each
  int n, r_max, s_max;
  struct Row {
    int d_res, d_tok, ent, d_chain, nb;   // nb = 2 r_max + 2
    __device__ __forceinline__ float at(int k) const {
      const bool one = (k == d_res) || (k == nb + d_tok) || (k == 2 * nb && ent) || (k == 2 * nb + 1 + d_chain);
      return one ? 1.0f : 0.0f;
    }
  };
  __device__ __forceinline__ Row row(long long r) const {
    const long long bi = r / n;                       // batch * n + i
    const long long bj = (bi / n) * n + (r - bi * n); // batch * n + j
    const bool chain = asym[bi] == asym[bj], res = residue[bi] == residue[bj], ent = entity[bi] == entity[bj];
    auto clip = [](long long d, int mx) { return static_cast<int>(d < 0 ? 0 : (d > 2 * mx ? 2 * mx : d)); };
    Row o;
    o.nb = 2 * r_max + 2;
    o.d_res = chain ? clip(residue[bi] - residue[bj] + r_max, r_max) : 2 * r_max + 1;
    o.d_tok = (chain && res) ? clip(token[bi] - token[bj] + r_max, r_max) : 2 * r_max + 1;
    o.ent = ent ? 1 : 0;
    o.d_chain = ent ? clip(sym[bi] - sym[bj] + s_max, s_max) : 2 * s_max + 1;
    return o;
  }
};

template <typename TZ, typename FEAT>
__global__ void __launch_bounds__(256) concat_layernorm_kernel(const TZ* __restrict__ z, const FEAT feat,
                                                               const float* __restrict__ w, const float* __restrict__ b,
                                                               float* __restrict__ y, long long rows, int c1, int c2, int k_pad,
                                                               float eps) {
  const int lane = threadIdx.x & 31;
  const int c = c1 + c2;
  const long long stride = static_cast<long long>(gridDim.x) * 8;
  for (long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5); row < rows; row += stride) {
    const TZ* zr = z + row * c1;
    const auto fr = feat.row(row);
    float v[kCatPerLane];
    float sum = 0.f;
#pragma unroll
    for (int g = 0; g < kCatPerLane; ++g) {
      const int ch = g * 32 + lane;
      v[g] = ch < c1 ? ldf(zr + ch) : (ch < c ? fr.at(ch - c1) : 0.f);
      sum += v[g];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / static_cast<float>(c);
    float sq = 0.f;
#pragma unroll
    for (int g = 0; g < kCatPerLane; ++g) {
      const float d = (g * 32 + lane) < c ? v[g] - mean : 0.f;
      sq = fmaf(d, d, sq);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = rsqrtf(sq / static_cast<float>(c) + eps);
    float* yr = y + row * k_pad;
#pragma unroll
    for (int g = 0; g < kCatPerLane; ++g) {
      const int ch = g * 32 + lane;
      if (ch < c) {
        float o = (v[g] - mean) * rstd;
        if (w != nullptr) o *= w[ch];
        if (b != nullptr) o += b[ch];
        yr[ch] = o;
      } else if (ch < k_pad) {
        yr[ch] = 0.f;
      }
    }
  }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) gelu_kernel(const TI* __restrict__ x, TO* __restrict__ y, long long n) {
  const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= n) return;
  const float v = ldf(x + i);
  stf(y + i, 0.5f * v * (1.0f + erff(v * 0.70710678118654752f)));
}

// out[b, i, j, :] = z[b, i, j, :] + row_add[b, j, :] + col_add[b, i, :]   (the single representation projected twice and
// added along the two token axes).  Four channels per thread.
template <typename T>
__global__ void __launch_bounds__(256) pair_outer_add_kernel(const T* __restrict__ z, const T* __restrict__ row_add,
                                                             const T* __restrict__ col_add, T* __restrict__ out, long long total,
                                                             int n, int c) {
  const long long e = (static_cast<long long>(blockIdx.x) * 256 + threadIdx.x) * 4;
  if (e >= total) return;
  const long long pos = e / c;
  const int ch = static_cast<int>(e - pos * c);
  const long long bi = pos / n;
  const int j = static_cast<int>(pos - bi * n);
  const long long b = bi / n;
#pragma unroll
  for (int k = 0; k < 4; ++k)
    stf(out + e + k, ldf(z + e + k) + ldf(row_add + (b * n + j) * c + ch + k) + ldf(col_add + bi * c + ch + k));
}

// out[b, i, j, :] = z[b, i, j, :] + w_t[bin(|x_i - x_j|), :], bin = number of boundaries below the distance: the one-hot
// distogram of the predicted structure embedded and added to the pair tensor.  x fp32 (b, n, 3); w_t (bins, c).
template <typename T>
__global__ void __launch_bounds__(256) distogram_embed_add_kernel(const T* __restrict__ z, const float* __restrict__ x,
                                                                  const float* __restrict__ boundaries, int n_bound,
                                                                  const T* __restrict__ w_t, T* __restrict__ out, int n, int c) {
  const long long pos = blockIdx.x;                     // (b * n + i) * n + j
  const long long bi = pos / n;
  const int j = static_cast<int>(pos - bi * n);
  const long long b = bi / n;
  const float* xi = x + bi * 3;
  const float* xj = x + (b * n + j) * 3;
  const float dx = xi[0] - xj[0], dy = xi[1] - xj[1], dz = xi[2] - xj[2];
  const float d = sqrtf(dx * dx + dy * dy + dz * dz);
  int bin = 0;
  for (int k = 0; k < n_bound; ++k) bin += d > boundaries[k] ? 1 : 0;
  for (int ch = threadIdx.x; ch < c; ch += 256) stf(out + pos * c + ch, ldf(z + pos * c + ch) + ldf(w_t + static_cast<long long>(bin) * c + ch));
}

}  // namespace

extern "C" {

KFB_API int kfb_pair_outer_add(const void* z, const void* row_add, const void* col_add, void* out, int batch, int n, int c, int dtype,
                               void* stream_) {
  KFB_CHECK_ARG(z && row_add && col_add && out, "pair_outer_add: null pointer");
  KFB_CHECK_ARG(batch >= 1 && n >= 1 && c >= 4 && c % 4 == 0, "pair_outer_add: batch %d n %d c %d (c a multiple of 4)", batch, n, c);
  KFB_CHECK_ARG(dtype == KFB_BF16 || dtype == KFB_FP32, "pair_outer_add: dtype %d", dtype);
  cudaStream_t stream = as_stream(stream_);
  const long long total = static_cast<long long>(batch) * n * n * c;
  const unsigned blocks = static_cast<unsigned>((total / 4 + 255) / 256);
  {
    LaunchScope scope(stream, "pair_outer_add");
    if (dtype == KFB_BF16)
      pair_outer_add_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(z), static_cast<const __nv_bfloat16*>(row_add),
                                                        static_cast<const __nv_bfloat16*>(col_add), static_cast<__nv_bfloat16*>(out), total, n, c);
    else
      pair_outer_add_kernel<<<blocks, 256, 0, stream>>>(static_cast<const float*>(z), static_cast<const float*>(row_add),
                                                        static_cast<const float*>(col_add), static_cast<float*>(out), total, n, c);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

KFB_API int kfb_distogram_embed_add(const void* z, const float* x, const float* boundaries, int n_boundaries, const void* w_t, void* out,
                                    int batch, int n, int c, int dtype, void* stream_) {
  KFB_CHECK_ARG(z && x && boundaries && w_t && out, "distogram_embed_add: null pointer");
  KFB_CHECK_ARG(batch >= 1 && n >= 1 && c >= 1 && n_boundaries >= 1 && static_cast<long long>(batch) * n * n < (1ll << 31),
                "distogram_embed_add: batch %d n %d c %d boundaries %d", batch, n, c, n_boundaries);
  KFB_CHECK_ARG(dtype == KFB_BF16 || dtype == KFB_FP32, "distogram_embed_add: dtype %d", dtype);
  cudaStream_t stream = as_stream(stream_);
  const unsigned blocks = static_cast<unsigned>(static_cast<long long>(batch) * n * n);
  {
    LaunchScope scope(stream, "distogram_embed_add");
    if (dtype == KFB_BF16)
      distogram_embed_add_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(z), x, boundaries, n_boundaries,
                                                             static_cast<const __nv_bfloat16*>(w_t), static_cast<__nv_bfloat16*>(out), n, c);
    else
      distogram_embed_add_kernel<<<blocks, 256, 0, stream>>>(static_cast<const float*>(z), x, boundaries, n_boundaries,
                                                             static_cast<const float*>(w_t), static_cast<float*>(out), n, c);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

KFB_API size_t kfb_parcae_workspace_bytes(long long rows, int c) { return align_up(static_cast<size_t>(rows) * c * 2, 256); }

KFB_API int kfb_parcae_fwd(const void* z, const void* u, const float* ln_w, const float* ln_b, const float* a, const void* b_w,
                           void* out, void* workspace, size_t workspace_bytes, long long rows, int c, float eps, int dtype,
                           void* stream_) {
  KFB_CHECK_ARG(z && u && a && b_w && out && workspace, "parcae: null pointer");
  KFB_CHECK_ARG(dtype == KFB_BF16 || dtype == KFB_FP32, "parcae: dtype %d (bf16 arithmetic on bf16 or fp32 tensors)", dtype);
  KFB_CHECK_ARG(rows >= 1 && rows < (1ll << 31) && c % 8 == 0 && c >= 32 && c <= 1024, "parcae: rows %lld c %d", rows, c);
  KFB_CHECK_ARG(workspace_bytes >= kfb_parcae_workspace_bytes(rows, c), "parcae: workspace too small");
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "parcae: workspace must be 256-byte aligned");
  cudaStream_t stream = as_stream(stream_);
  __nv_bfloat16* xn = static_cast<__nv_bfloat16*>(workspace);
  KFB_TRY(launch_layernorm(stream, u, xn, ln_w, ln_b, rows, c, c, c, eps, dtype, KFB_BF16));
  GemmParams p = {};
  p.n_extent = static_cast<int>(rows);
  p.o_extent = 1;
  p.batch = 1;
  p.n_cols = c;
  p.k_extent = c;
  p.nseg = 1;
  p.seg[0] = row_major_seg(out, c, c, 0, 0, dtype == KFB_FP32);
  p.resid = z;
  p.resid_scale = a;
  GemmOperandA oa = {xn, c, 0, 0};
  GemmOperandB ob = {b_w, c, 0};
  return launch_gemm_bf16(stream, oa, ob, p, 0, "parcae_update");
}

KFB_API int kfb_lm_pair_features(const void* x, void* out, int batch, int n, int d, int dtype, void* stream_) {
  KFB_CHECK_ARG(x && out, "lm_pair_features: null pointer");
  KFB_CHECK_ARG(batch >= 1 && n >= 1 && d >= 1 && static_cast<long long>(batch) * n < (1ll << 31), "lm_pair_features: batch %d n %d d %d",
                batch, n, d);
  KFB_CHECK_ARG(dtype == KFB_BF16 || dtype == KFB_FP32, "lm_pair_features: dtype %d", dtype);
  cudaStream_t stream = as_stream(stream_);
  {
    LaunchScope scope(stream, "lm_pair_features");
    if (dtype == KFB_BF16)
      lm_pair_features_kernel<__nv_bfloat16><<<batch * n, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                                            static_cast<__nv_bfloat16*>(out), n, d);
    else
      lm_pair_features_kernel<float><<<batch * n, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<__nv_bfloat16*>(out), n, d);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

KFB_API int kfb_concat_layernorm(const void* z, int z_dtype, const void* rel, int rel_dtype, const float* ln_w, const float* ln_b,
                                 float* out, long long rows, int c1, int c2, int k_pad, float eps, void* stream_) {
  KFB_CHECK_ARG(z && rel && out && rows >= 1, "concat_layernorm: null pointer or empty tensor");
  KFB_CHECK_ARG(c1 >= 1 && c2 >= 1 && k_pad >= c1 + c2 && k_pad <= 32 * kCatPerLane,
                "concat_layernorm: %d + %d channels padded to %d (at most %d)", c1, c2, k_pad, 32 * kCatPerLane);
  KFB_CHECK_ARG((z_dtype == KFB_BF16 || z_dtype == KFB_FP32) && (rel_dtype == KFB_BF16 || rel_dtype == KFB_FP32),
                "concat_layernorm: dtypes %d %d", z_dtype, rel_dtype);
  cudaStream_t stream = as_stream(stream_);
  long long blocks = (rows + 7) / 8;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  const unsigned g = static_cast<unsigned>(blocks);
  {
    LaunchScope scope(stream, "concat_layernorm");
    const StoredFeatures<__nv_bfloat16> fb = {static_cast<const __nv_bfloat16*>(rel), c2};
    const StoredFeatures<float> ff = {static_cast<const float*>(rel), c2};
    if (z_dtype == KFB_BF16 && rel_dtype == KFB_BF16)
      concat_layernorm_kernel<<<g, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(z), fb, ln_w, ln_b, out, rows, c1, c2, k_pad, eps);
    else if (z_dtype == KFB_BF16)
      concat_layernorm_kernel<<<g, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(z), ff, ln_w, ln_b, out, rows, c1, c2, k_pad, eps);
    else if (rel_dtype == KFB_BF16)
      concat_layernorm_kernel<<<g, 256, 0, stream>>>(static_cast<const float*>(z), fb, ln_w, ln_b, out, rows, c1, c2, k_pad, eps);
    else
      concat_layernorm_kernel<<<g, 256, 0, stream>>>(static_cast<const float*>(z), ff, ln_w, ln_b, out, rows, c1, c2, k_pad, eps);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

KFB_API int kfb_relpos_concat_layernorm(const void* z, int z_dtype, const long long* asym_id, const long long* residue_index,
                                        const long long* entity_id, const long long* token_index, const long long* sym_id,
                                        int r_max, int s_max, const float* ln_w, const float* ln_b, float* out, int batch, int n, int c1,
                                        int k_pad, float eps, void* stream_) {
  KFB_CHECK_ARG(z && asym_id && residue_index && entity_id && token_index && sym_id && out, "relpos_concat_layernorm: null pointer");
  KFB_CHECK_ARG(batch >= 1 && n >= 1 && c1 >= 1 && r_max >= 0 && s_max >= 0, "relpos_concat_layernorm: bad sizes");
  const int c2 = 4 * (r_max + 1) + 2 * (s_max + 1) + 1;
  KFB_CHECK_ARG(k_pad >= c1 + c2 && k_pad <= 32 * kCatPerLane, "relpos_concat_layernorm: %d + %d channels padded to %d (at most %d)", c1,
                c2, k_pad, 32 * kCatPerLane);
  KFB_CHECK_ARG(z_dtype == KFB_BF16 || z_dtype == KFB_FP32, "relpos_concat_layernorm: dtype %d", z_dtype);
  cudaStream_t stream = as_stream(stream_);
  const long long rows = static_cast<long long>(batch) * n * n;
  long long blocks = (rows + 7) / 8;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  const RelPosFeatures feat = {asym_id, residue_index, entity_id, token_index, sym_id, n, r_max, s_max};
  {
    LaunchScope scope(stream, "relpos_concat_layernorm");
    if (z_dtype == KFB_BF16)
      concat_layernorm_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(z), feat, ln_w, ln_b,
                                                                                  out, rows, c1, c2, k_pad, eps);
    else
      concat_layernorm_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const float*>(z), feat, ln_w, ln_b, out,
                                                                                  rows, c1, c2, k_pad, eps);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

KFB_API int kfb_gelu(const void* x, void* y, long long n, int in_dtype, int out_dtype, void* stream_) {
  KFB_CHECK_ARG(x && y && n >= 1, "gelu: null pointer or empty tensor");
  KFB_CHECK_ARG((in_dtype == KFB_BF16 || in_dtype == KFB_FP32) && (out_dtype == KFB_BF16 || out_dtype == KFB_FP32), "gelu: dtypes %d %d",
                in_dtype, out_dtype);
  cudaStream_t stream = as_stream(stream_);
  const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
  {
    LaunchScope scope(stream, "gelu");
    if (in_dtype == KFB_BF16 && out_dtype == KFB_BF16)
      gelu_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n);
    else if (in_dtype == KFB_BF16)
      gelu_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<float*>(y), n);
    else if (out_dtype == KFB_BF16)
      gelu_kernel<<<blocks, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<__nv_bfloat16*>(y), n);
    else
      gelu_kernel<<<blocks, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<float*>(y), n);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

}  // extern "C"
