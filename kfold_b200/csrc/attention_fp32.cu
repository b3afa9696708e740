// fp32 attention with pair bias and key mask for the fp32-accurate mode.
//
// Plain CUDA cores, one query row per thread, keys streamed through shared memory in tiles of 32 with an
// online softmax (the L x L x H logits are never stored).  It exists for parity at fp32 accuracy, not for
// speed: the bf16 tensor-core kernel in attention.cu is the production path.  Same semantics: additive pair
// bias, masked keys get -1e9 (finite, as the reference does), optional sigmoid gate, and the result is written
// as the bf16 triple split [o0 o0 o1 o1 o0 o2] that the fp32-accurate output projection consumes.
#include "attention.cuh"
#include "ptx.cuh"

namespace kfb {

static constexpr int kFq = 128;  // queries per block (one per thread)
static constexpr int kFk = 32;   // keys per tile

template <int D>
__global__ void __launch_bounds__(kFq) attention_fp32_kernel(const AttnFp32Params p) {
  __shared__ float s_k[kFk][D + 1];
  __shared__ float s_v[kFk][D + 1];
  __shared__ float s_bias[kFq][kFk + 1];
  __shared__ float s_mask[kFk];
  const int tid = threadIdx.x;
  const int qb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q_idx = qb * kFq + tid;
  const bool q_ok = q_idx < p.lq;
  const long long qrow = static_cast<long long>(b) * p.lq + (q_ok ? q_idx : 0);
  float q[D], acc[D];
#pragma unroll
  for (int d = 0; d < D; ++d) {
    q[d] = p.q[qrow * p.ld + p.q_col0 + h * D + d];
    acc[d] = 0.f;
  }
  float m_run = -INFINITY, l_run = 0.f;
  const int b_hi = b / p.mask_lo_extent, b_lo = b - b_hi * p.mask_lo_extent;
  const unsigned char* mrow =
      p.mask == nullptr ? nullptr : p.mask + static_cast<long long>(b_hi) * p.m_hi + static_cast<long long>(b_lo) * p.m_lo;
  const int bias_b = p.bias_mod > 0 ? (b / p.bias_div) * p.bias_mod + b % p.bias_mod : b / p.bias_div;
  const long long bias_z = p.bias_head_major > 0 ? static_cast<long long>(h) * p.bias_head_major + bias_b
                                                 : static_cast<long long>(bias_b) * p.heads + h;
  const float* bias_base = p.bias + bias_z * static_cast<long long>(p.lq) * p.ldb;
  const long long ld_kv = p.ld_kv > 0 ? p.ld_kv : p.ld;

  for (int k0 = 0; k0 < p.lk; k0 += kFk) {
    __syncthreads();
    // K and V tiles: kFk keys x D values each
    for (int idx = tid; idx < kFk * D; idx += kFq) {
      const int kk = idx / D, d = idx - kk * D;
      const int key = k0 + kk;
      float kv = 0.f, vv = 0.f;
      if (key < p.lk) {
        const long long krow = static_cast<long long>(b) * p.lk + key;
        kv = p.k[krow * ld_kv + p.k_col0 + h * D + d];
        vv = p.v[krow * ld_kv + p.v_col0 + h * D + d];
      }
      s_k[kk][d] = kv;
      s_v[kk][d] = vv;
    }
    // bias tile: kFq queries x kFk keys
    for (int idx = tid; idx < kFq * kFk; idx += kFq) {
      const int qq = idx / kFk, kk = idx - qq * kFk;
      const int qi = qb * kFq + qq, key = k0 + kk;
      s_bias[qq][kk] = (qi < p.lq && key < p.lk) ? bias_base[static_cast<long long>(qi) * p.ldb + key] : 0.f;
    }
    if (tid < kFk) {
      const int key = k0 + tid;
      s_mask[tid] = key < p.lk ? ((mrow == nullptr || mrow[static_cast<long long>(key) * p.m_k]) ? 0.f : -1e9f) : -INFINITY;
    }
    __syncthreads();
    float s[kFk];
    float mx = -INFINITY;
#pragma unroll
    for (int kk = 0; kk < kFk; ++kk) {
      float dot = 0.f;
#pragma unroll
      for (int d = 0; d < D; ++d) dot = fmaf(q[d], s_k[kk][d], dot);
      // same order of additions as the reference: (q k + mask) + bias
      s[kk] = (dot + s_mask[kk]) + s_bias[tid][kk];
      mx = fmaxf(mx, s[kk]);
    }
    const float m_new = fmaxf(m_run, mx);
    const float alpha = expf(m_run - m_new);
    l_run *= alpha;
#pragma unroll
    for (int d = 0; d < D; ++d) acc[d] *= alpha;
#pragma unroll
    for (int kk = 0; kk < kFk; ++kk) {
      const float pr = expf(s[kk] - m_new);
      l_run += pr;
#pragma unroll
      for (int d = 0; d < D; ++d) acc[d] = fmaf(pr, s_v[kk][d], acc[d]);
    }
    m_run = m_new;
  }
  if (!q_ok) return;
  const float inv_l = 1.0f / l_run;
  const int hd = p.heads * D;
  __nv_bfloat16* o6 = p.out6 + qrow * 6 * hd;
#pragma unroll
  for (int d = 0; d < D; ++d) {
    float o = acc[d] * inv_l;
    if (p.g != nullptr) o *= 1.0f / (1.0f + expf(-p.g[qrow * p.ld + p.g_col0 + h * D + d]));
    const int col = h * D + d;
    const __nv_bfloat16 x0 = __float2bfloat16_rn(o);
    const float r1 = o - __bfloat162float(x0);
    const __nv_bfloat16 x1 = __float2bfloat16_rn(r1);
    const __nv_bfloat16 x2 = __float2bfloat16_rn(r1 - __bfloat162float(x1));
    o6[col] = x0; o6[hd + col] = x0; o6[2 * hd + col] = x1; o6[3 * hd + col] = x1; o6[4 * hd + col] = x0; o6[5 * hd + col] = x2;
  }
}

int launch_attention_fp32(cudaStream_t stream, const AttnFp32Params& p) {
  KFB_CHECK_ARG(p.batch > 0 && p.heads > 0 && p.lq > 0 && p.lk > 0, "attention_fp32: empty problem");
  KFB_CHECK_ARG(p.batch <= 65535 && p.heads <= 65535, "attention_fp32: batch %d / heads %d exceed the grid limits", p.batch, p.heads);
  dim3 grid(cdiv(p.lq, kFq), p.heads, p.batch);
  LaunchScope scope(stream, p.tag ? p.tag : "attention_fp32");
  switch (p.d) {
    case 16: attention_fp32_kernel<16><<<grid, kFq, 0, stream>>>(p); break;
    case 24: attention_fp32_kernel<24><<<grid, kFq, 0, stream>>>(p); break;
    case 32: attention_fp32_kernel<32><<<grid, kFq, 0, stream>>>(p); break;
    case 48: attention_fp32_kernel<48><<<grid, kFq, 0, stream>>>(p); break;
    case 64: attention_fp32_kernel<64><<<grid, kFq, 0, stream>>>(p); break;
    default:
      set_error("attention_fp32: head dim %d not supported (16, 24, 32, 48, 64)", p.d);
      return KFB_ERR_UNSUPPORTED;
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

}  // namespace kfb
