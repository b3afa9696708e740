// Flash-style pair-bias attention kernel (see attention.cuh for the contract).
#include <cuda_bf16.h>

#include <mutex>

#include "attention.cuh"
#include "gemm.cuh"  // sigmoidf_fast, pack_bf16x2
#include "ptx.cuh"

namespace kfb {

static constexpr int kAttThreads = 192;
static constexpr int kBQ = 128;   // queries per CTA
static constexpr int kBKV = 128;  // keys per block
static constexpr float kLog2e = 1.4426950408889634f;
static constexpr float kMaskInf = 1e9f;

template <int DPAD>
struct AttCfg {
  static constexpr int kSpan = DPAD * 2;                 // bytes per q/k row = swizzle span
  static constexpr int kQBytes = kBQ * kSpan;
  static constexpr int kKBytes = kBKV * kSpan;
  static constexpr int kVBytes = 2 * DPAD * 128;         // two boxes of [DPAD rows x 64 keys]
  static constexpr int kKvStages = 2;
  static constexpr int kBiasBytes = 2 * kBQ * 128;       // two boxes of [128 rows x 64 keys] bf16
  static constexpr int kPBytes = 2 * kBQ * 128;
  static constexpr int kTmemCols = 256;                  // S: 128 columns, O: DPAD columns at offset 128
  static constexpr int kSmemBytes = kQBytes + kKvStages * (kKBytes + kVBytes) + kBiasBytes + kPBytes + 1024 /*align*/ +
                                    2 * kBKV * 4 /*mask*/ + 256 /*barriers*/;
};

template <int DPAD>
__global__ void __launch_bounds__(kAttThreads, 1)
attention_bias_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_b,
                      const AttnParams p) {
  using Cfg = AttCfg<DPAD>;
  constexpr int kStages = Cfg::kKvStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem;
  uint8_t* s_k = s_q + Cfg::kQBytes;
  uint8_t* s_v = s_k + kStages * Cfg::kKBytes;
  uint8_t* s_bias = s_v + kStages * Cfg::kVBytes;
  uint8_t* s_p = s_bias + Cfg::kBiasBytes;
  float* s_mask = reinterpret_cast<float*>(s_p + Cfg::kPBytes);  // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_mask + 2 * kBKV);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;            // [kStages]
  uint64_t* kv_empty = kv_full + kStages;  // [kStages]
  uint64_t* bias_full = kv_empty + kStages;
  uint64_t* bias_empty = bias_full + 1;
  uint64_t* s_full = bias_empty + 1;
  uint64_t* s_empty = s_full + 1;
  uint64_t* p_full = s_empty + 1;
  uint64_t* o_full = p_full + 1;
  uint64_t* mask_bar = o_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mask_bar + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qb = blockIdx.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int nkv = (p.lk + kBKV - 1) / kBKV;

  if (threadIdx.x == 0) {
    ptx::prefetch_tmap(&tm_q);
    ptx::prefetch_tmap(&tm_k);
    ptx::prefetch_tmap(&tm_v);
    ptx::prefetch_tmap(&tm_b);
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&kv_full[s], 1);
      ptx::mbar_init(&kv_empty[s], 1);
    }
    ptx::mbar_init(bias_full, 1);
    ptx::mbar_init(bias_empty, 128);
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(s_empty, 128);
    ptx::mbar_init(p_full, 128);
    ptx::mbar_init(o_full, 1);
    ptx::mbar_init(mask_bar, 128);
    ptx::fence_barrier_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_o = tmem_base + 128;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      ptx::mbar_expect_tx(q_full, Cfg::kQBytes);
      ptx::tma_load_3d(s_q, &tm_q, q_full, p.q_col0 + h * DPAD, qb * kBQ, b);
      const int bias_z = (b / p.bias_div) * p.heads + h;
      for (int j = 0; j < nkv; ++j) {
        const int st = j % kStages;
        if (!ptx::mbar_wait(&kv_empty[st], ((j / kStages) & 1) ^ 1, 201)) break;
        ptx::mbar_expect_tx(&kv_full[st], Cfg::kKBytes + Cfg::kVBytes);
        ptx::tma_load_3d(s_k + st * Cfg::kKBytes, &tm_k, &kv_full[st], p.k_col0 + h * DPAD, j * kBKV, b);
        ptx::tma_load_3d(s_v + st * Cfg::kVBytes, &tm_v, &kv_full[st], j * kBKV, h * DPAD, b);
        ptx::tma_load_3d(s_v + st * Cfg::kVBytes + DPAD * 128, &tm_v, &kv_full[st], j * kBKV + 64, h * DPAD, b);
        if (!ptx::mbar_wait(bias_empty, (j & 1) ^ 1, 202)) break;
        ptx::mbar_expect_tx(bias_full, Cfg::kBiasBytes);
        ptx::tma_load_3d(s_bias, &tm_b, bias_full, j * kBKV, qb * kBQ, bias_z);
        ptx::tma_load_3d(s_bias + kBQ * 128, &tm_b, bias_full, j * kBKV + 64, qb * kBQ, bias_z);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = ptx::make_idesc(kBQ, kBKV, 1);
      constexpr uint32_t idesc_o = ptx::make_idesc(kBQ, DPAD, 1);
      bool ok = ptx::mbar_wait(q_full, 0, 203);
      const uint32_t q_addr = ptx::smem_u32(s_q);
      const uint32_t p_addr = ptx::smem_u32(s_p);
      for (int j = 0; ok && j < nkv; ++j) {
        const int st = j % kStages;
        if (!ptx::mbar_wait(&kv_full[st], (j / kStages) & 1, 204)) break;
        if (!ptx::mbar_wait(s_empty, (j & 1) ^ 1, 205)) break;
        ptx::tc_fence_after_sync();
        const uint32_t k_addr = ptx::smem_u32(s_k + st * Cfg::kKBytes);
#pragma unroll
        for (int kk = 0; kk < DPAD / 16; ++kk)
          ptx::mma_f16_ss(tmem_s, ptx::make_kmajor_desc<Cfg::kSpan>(q_addr + kk * 32),
                          ptx::make_kmajor_desc<Cfg::kSpan>(k_addr + kk * 32), idesc_s, kk != 0 ? 1u : 0u);
        ptx::tc_commit(s_full);
        if (!ptx::mbar_wait(p_full, j & 1, 206)) break;
        ptx::tc_fence_after_sync();
        const uint32_t v_addr = ptx::smem_u32(s_v + st * Cfg::kVBytes);
#pragma unroll
        for (int kk = 0; kk < kBKV / 16; ++kk) {
          const uint32_t pa = p_addr + (kk >> 2) * (kBQ * 128) + (kk & 3) * 32;
          const uint32_t va = v_addr + (kk >> 2) * (DPAD * 128) + (kk & 3) * 32;
          ptx::mma_f16_ss(tmem_o, ptx::make_kmajor_desc<128>(pa), ptx::make_kmajor_desc<128>(va), idesc_o,
                          kk != 0 ? 1u : 0u);
        }
        ptx::tc_commit(o_full);
        ptx::tc_commit(&kv_empty[st]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + accumulation (warps 2..5)
    const int quad = warp & 3;
    const int r = quad * 32 + lane;   // row inside the query block == TMEM lane
    const int sm_tid = threadIdx.x - 64;  // 0..127
    const int q_idx = qb * kBQ + r;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int b_hi = b / p.mask_lo_extent, b_lo = b - b_hi * p.mask_lo_extent;
    const unsigned char* mrow = p.mask + static_cast<long long>(b_hi) * p.m_hi + static_cast<long long>(b_lo) * p.m_lo;

    float acc[DPAD];
#pragma unroll
    for (int i = 0; i < DPAD; ++i) acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;

    for (int j = 0; j < nkv; ++j) {
      // additive key mask of this block, shared by all rows of the CTA
      {
        const int key = j * kBKV + sm_tid;
        float mv = -INFINITY;  // keys beyond lk do not exist
        if (key < p.lk) mv = mrow[static_cast<long long>(key) * p.m_k] ? 0.f : -kMaskInf;
        s_mask[(j & 1) * kBKV + sm_tid] = mv;
      }
      // a bounded mbarrier instead of bar.sync: a thread that gave up elsewhere can never strand the others here
      ptx::mbar_arrive(mask_bar);
      if (!ptx::mbar_wait(mask_bar, j & 1, 211)) { ok = false; break; }
      const float* mk = s_mask + (j & 1) * kBKV;
      if (!ptx::mbar_wait(s_full, j & 1, 207)) { ok = false; break; }
      if (!ptx::mbar_wait(bias_full, j & 1, 208)) { ok = false; break; }
      ptx::tc_fence_after_sync();

      // ---- pass 1: row maximum of (S + mask + bias) in log2 units
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t raw[32];
        ptx::tmem_ld_32x32b_x32(tmem_s + lane_base + c * 32, raw);
        const uint8_t* brow = s_bias + (c >> 1) * (kBQ * 128) + r * 128;
        float bv[32];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ci = ((c & 1) * 4 + i) ^ (r & 7);
          const uint4 u = *reinterpret_cast<const uint4*>(brow + (ci << 4));
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[t]));
            bv[i * 8 + t * 2] = f.x;
            bv[i * 8 + t * 2 + 1] = f.y;
          }
        }
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float t = ((__uint_as_float(raw[i]) + mk[c * 32 + i]) + bv[i]) * kLog2e;
          mx = fmaxf(mx, t);
        }
      }
      const float m_new = fmaxf(m_run, mx);
      const float alpha = exp2f(m_run - m_new);  // m_run = -inf on the first block -> 0
      // ---- fold the previous block's P V product (still in the previous scale) and rescale
      if (j > 0) {
        if (!ptx::mbar_wait(o_full, (j - 1) & 1, 209)) { ok = false; break; }
        ptx::tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < DPAD / 32; ++c) {
          uint32_t raw[32];
          ptx::tmem_ld_32x32b_x32(tmem_o + lane_base + c * 32, raw);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c * 32 + i] = (acc[c * 32 + i] + __uint_as_float(raw[i])) * alpha;
        }
      }
      l_run *= alpha;
      // ---- pass 2: P = exp2(t - m_new), written as bf16 into the swizzled A-operand tile
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t raw[32];
        ptx::tmem_ld_32x32b_x32(tmem_s + lane_base + c * 32, raw);
        const uint8_t* brow = s_bias + (c >> 1) * (kBQ * 128) + r * 128;
        uint8_t* prow = s_p + (c >> 1) * (kBQ * 128) + r * 128;
        float bv[32];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ci = ((c & 1) * 4 + i) ^ (r & 7);
          const uint4 u = *reinterpret_cast<const uint4*>(brow + (ci << 4));
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[t]));
            bv[i * 8 + t * 2] = f.x;
            bv[i * 8 + t * 2 + 1] = f.y;
          }
        }
        ptx::tmem_ld_wait();
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float t = ((__uint_as_float(raw[i]) + mk[c * 32 + i]) + bv[i]) * kLog2e;
          pv[i] = exp2f(t - m_new);
          l_run += pv[i];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ci = ((c & 1) * 4 + i) ^ (r & 7);
          *reinterpret_cast<uint4*>(prow + (ci << 4)) =
              make_uint4(pack_bf16x2(pv[i * 8], pv[i * 8 + 1]), pack_bf16x2(pv[i * 8 + 2], pv[i * 8 + 3]),
                         pack_bf16x2(pv[i * 8 + 4], pv[i * 8 + 5]), pack_bf16x2(pv[i * 8 + 6], pv[i * 8 + 7]));
        }
      }
      m_run = m_new;
      ptx::tc_fence_before_sync();
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(p_full);
      ptx::mbar_arrive(s_empty);
      ptx::mbar_arrive(bias_empty);
    }
    if (ok && ptx::mbar_wait(o_full, (nkv - 1) & 1, 210)) {
      ptx::tc_fence_after_sync();
      const float inv_l = 1.0f / l_run;
#pragma unroll
      for (int c = 0; c < DPAD / 32; ++c) {
        uint32_t raw[32];
        ptx::tmem_ld_32x32b_x32(tmem_o + lane_base + c * 32, raw);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[c * 32 + i] = (acc[c * 32 + i] + __uint_as_float(raw[i])) * inv_l;
      }
      if (q_idx < p.lq) {
        const long long row = static_cast<long long>(b) * p.lq + q_idx;
        if (p.g != nullptr) {
          const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(p.g) + row * p.ldg + p.g_col0 + h * DPAD;
#pragma unroll
          for (int i = 0; i < DPAD; i += 8) {
            const uint4 u = *reinterpret_cast<const uint4*>(g + i);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[t]));
              acc[i + t * 2] *= sigmoidf_fast(f.x);
              acc[i + t * 2 + 1] *= sigmoidf_fast(f.y);
            }
          }
        }
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.ldo + h * p.d;
#pragma unroll
        for (int i = 0; i < DPAD; i += 8) {
          if (i < p.d)  // d is a multiple of 8
            *reinterpret_cast<uint4*>(o + i) =
                make_uint4(pack_bf16x2(acc[i], acc[i + 1]), pack_bf16x2(acc[i + 2], acc[i + 3]),
                           pack_bf16x2(acc[i + 4], acc[i + 5]), pack_bf16x2(acc[i + 6], acc[i + 7]));
        }
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int DPAD>
static int launch_dpad(cudaStream_t stream, const AttnParams& p) {
  using Cfg = AttCfg<DPAD>;
  static std::once_flag once[64];
  int dev = 0;
  KFB_CUDA(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  std::call_once(once[dev & 63], [&] {
    attr_err = cudaFuncSetAttribute(attention_bias_kernel<DPAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  });
  KFB_CUDA(attr_err);
  CUtensorMap tq, tk, tv, tb;
  {
    const uint64_t dims[3] = {(uint64_t)p.ldq, (uint64_t)p.lq, (uint64_t)p.batch};
    const uint64_t str[2] = {(uint64_t)p.ldq * 2, (uint64_t)p.lq * p.ldq * 2};
    const uint32_t box[3] = {DPAD, kBQ, 1};
    KFB_TRY(make_tmap(&tq, p.q, 2, 3, dims, str, box, Cfg::kSpan));
  }
  {
    const uint64_t dims[3] = {(uint64_t)p.ldk, (uint64_t)p.lk, (uint64_t)p.batch};
    const uint64_t str[2] = {(uint64_t)p.ldk * 2, (uint64_t)p.lk * p.ldk * 2};
    const uint32_t box[3] = {DPAD, kBKV, 1};
    KFB_TRY(make_tmap(&tk, p.k, 2, 3, dims, str, box, Cfg::kSpan));
  }
  {
    const uint64_t dims[3] = {(uint64_t)p.lk, (uint64_t)p.heads * DPAD, (uint64_t)p.batch};
    const uint64_t str[2] = {(uint64_t)p.ldv * 2, (uint64_t)p.heads * DPAD * p.ldv * 2};
    const uint32_t box[3] = {64, DPAD, 1};
    KFB_TRY(make_tmap(&tv, p.vt, 2, 3, dims, str, box, 128));
  }
  {
    const int bias_batches = cdiv(p.batch, p.bias_div);
    const uint64_t dims[3] = {(uint64_t)p.lk, (uint64_t)p.lq, (uint64_t)bias_batches * p.heads};
    const uint64_t str[2] = {(uint64_t)p.ldb * 2, (uint64_t)p.lq * p.ldb * 2};
    const uint32_t box[3] = {64, kBQ, 1};
    KFB_TRY(make_tmap(&tb, p.bias, 2, 3, dims, str, box, 128));
  }
  dim3 grid(cdiv(p.lq, kBQ), p.heads, p.batch);
  {
    LaunchScope scope(stream, p.tag ? p.tag : "attention");
    attention_bias_kernel<DPAD><<<grid, kAttThreads, Cfg::kSmemBytes, stream>>>(tq, tk, tv, tb, p);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

int launch_attention(cudaStream_t stream, const AttnParams& p) {
  KFB_CHECK_ARG(p.batch > 0 && p.heads > 0 && p.lq > 0 && p.lk > 0, "attention: empty problem");
  KFB_CHECK_ARG(p.batch <= 65535 * 32, "attention: batch %d too large", p.batch);
  KFB_CHECK_ARG(p.d % 8 == 0 && p.d <= p.dpad, "attention: head dim %d must be a multiple of 8 and <= %d", p.d, p.dpad);
  KFB_CHECK_ARG(p.ldq % 8 == 0 && p.ldk % 8 == 0 && p.ldv % 8 == 0 && p.ldb % 8 == 0 && p.ldo % 8 == 0,
                "attention: leading dimensions must be multiples of 8 elements");
  KFB_CHECK_ARG(p.bias_div >= 1 && p.mask_lo_extent >= 1, "attention: bad divisors");
  KFB_CHECK_ARG(p.batch <= 65535, "attention: batch %d exceeds the grid z limit", p.batch);
  if (p.dpad == 32) return launch_dpad<32>(stream, p);
  if (p.dpad == 64) return launch_dpad<64>(stream, p);
  set_error("attention: padded head dim %d not supported (32 or 64)", p.dpad);
  return KFB_ERR_UNSUPPORTED;
}

}  // namespace kfb
