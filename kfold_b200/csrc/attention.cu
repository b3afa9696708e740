// Flash-style pair-bias attention kernel (see attention.cuh for the contract).
#include <cuda_bf16.h>

#include <mutex>

#include "attention.cuh"
#include "gemm.cuh"  // sigmoidf_fast, pack_bf16x2
#include "ptx.cuh"

namespace kfb {

static constexpr int kBQ = 128;   // queries per CTA
static constexpr int kBKV = 128;  // keys per block
static constexpr float kLog2e = 1.4426950408889634f;
// Logits are kept in log2 units: the packed query projection carries log2(e) / sqrt(D), the bias is multiplied by
// log2(e) as it is added, so that P = exp2(x - s) needs no further scaling and the subtraction is exact.
static constexpr float kMasked = -1e9f * 1.4426950408889634f;  // a masked key: the reference's finite -1e9, in log2 units
static constexpr float kAbsent = -1e30f;        // keys beyond lk
static constexpr float kRedoSum = 1.2676506e30f;  // 2^100: a half-tile row sum above this moves the stabiliser

template <int DPAD, int R>
struct AttCfg {
  // warp 0: TMA producer; warps 1..R: one MMA-issuing warp per row group (they sit on different schedulers, so
  // neither queues behind the other's waits); warp 3 (and 2 when R == 1): idle; then 8 softmax warps per row group
  static constexpr int kThreads = 128 + 256 * R;
  static constexpr int kSpan = DPAD * 2;                 // bytes per q/k row = swizzle span
  static constexpr int kQBytes = kBQ * kSpan;            // per row group
  static constexpr int kKBytes = kBKV * kSpan;
  static constexpr int kVBytes = 2 * DPAD * 128;         // two boxes of [DPAD rows x 64 keys]
  // one row group per CTA (R == 1) at head dim <= 32 is sized so that TWO CTAs fit an SM (shared memory <= 113 KB, 256
  // tensor-memory columns, 80 registers): two K/V stages there, three otherwise
  static constexpr bool kTwoPerSm = (R == 1 && DPAD == 32);
  static constexpr int kKvStages = kTwoPerSm ? 2 : 3;
  static constexpr int kTileBytes = 128 * 128;           // a bias half tile: 128 query rows x 64 keys bf16 (128-byte rows)
  static constexpr int kSmallBytes = 128 * 32;           // a 128 x 16 bf16 K-major operand without swizzle
  static constexpr int kBiasStages = 3;                  // ring of bias half tiles
  // tensor memory columns.  Keys are processed in half tiles of 64 (t = 0, 1, ...; buf = t % 3); the 64 columns
  // of a half tile are shared between two independent softmax streams (c = 0: keys 0..31, c = 1: keys 32..63):
  //   S[g][buf]  64 fp32 columns at (g*3 + buf) * 64; stream c overwrites the first 16 of its 32 columns
  //              with P (64 bf16 = 16 columns) in place, so a buffer is busy from S(t) until P V(t) has read it
  //   O[g][c]    DPAD fp32 columns at R*192 + (g*2 + c) * DPAD  (one accumulator per stream)
  static constexpr int kSBufs = 3;
  static constexpr int kTmemO = R * 192;
  static constexpr int kTmemUsed = R * (192 + 2 * DPAD);
  static constexpr int kTmemCols = kTmemUsed <= 256 ? 256 : 512;
  static constexpr int kXchgStride = DPAD + 3;           // floats per row of the end-of-kernel exchange (odd: no bank conflicts)
  static constexpr int kSmemBytes = R * kQBytes + R * kKvStages * (kKBytes + kVBytes) + kBiasStages * kTileBytes /*bias*/ +
                                    kSmallBytes /*e0*/ + R * 3 * kSmallBytes /*mask rows, three buffers*/ + 1024 /*align*/ +
                                    256 /*barriers*/;
};

// K-major operand without swizzle: 8 x 8 core matrices (8 rows of 16 bytes); the two K halves of a K=16
// slice are 128 bytes apart (leading byte offset), groups of 8 rows 256 bytes apart (stride byte offset).
__device__ __forceinline__ uint64_t make_noswizzle_desc(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4) | (static_cast<uint64_t>(128 >> 4) << 16) |
         (static_cast<uint64_t>(256 >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ uint32_t small_operand_row_offset(int r) { return (r >> 3) * 256 + (r & 7) * 16; }

// Pipeline.  A CTA owns 128 queries of R pair rows ("row groups", they share the bias tile).  Keys go by in half
// tiles of 64 (t = 0, 1, ...).  Each row group has two softmax streams of four warps: stream c owns 32 of the 64
// key columns of every half tile and keeps its own stabiliser, row sum and output accumulator O[g][c] (in tensor
// memory, accumulated by the tensor core); the two partial results are merged once at the end.
//   MMA warp g:  S(t) = Q K(t)^T + e0 maskrow(t)^T -> S[g][t % 3]                   commit s_full[g][t % 3]
//   stream c:    wait s_full; x = S_c(t) + bias_c(t) (own bias row from shared memory); P_c(t) = exp2(x - s) against a
//                lagging stabiliser, written over the stream's own S columns; arrive p_ready[g][t % 3] (both streams)
//   MMA warp g:  wait p_ready[g][t % 3] -> O[g][c] += P_c(t) V_c(t), then S(t+3) into the same buffer (the tensor
//                core executes in order, so S(t+3) cannot overtake the P V product that reads the buffer)
// S runs up to three half tiles ahead of the softmax, so the softmax warps never wait for the tensor core or for the
// issuing warp, and four independent softmax warps per scheduler hide each other's tensor-memory and MUFU latencies.
template <int DPAD, int R, bool WIN>
__global__ void __launch_bounds__(AttCfg<DPAD, R>::kThreads, AttCfg<DPAD, R>::kTwoPerSm ? 2 : 1)
attention_bias_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_b,
                      const AttnParams p) {
  using Cfg = AttCfg<DPAD, R>;
  constexpr int kStages = Cfg::kKvStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem;                                            // [R]
  uint8_t* s_k = s_q + R * Cfg::kQBytes;                          // [R][stages]
  uint8_t* s_v = s_k + R * kStages * Cfg::kKBytes;                // [R][stages]
  uint8_t* s_bias = s_v + R * kStages * Cfg::kVBytes;             // [stages][2 halves][128 rows][128 B]
  uint8_t* s_e0 = s_bias + Cfg::kBiasStages * Cfg::kTileBytes;
  uint8_t* s_maskrow = s_e0 + Cfg::kSmallBytes;                   // [R][3]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_maskrow + R * 3 * Cfg::kSmallBytes);
  uint64_t* q_full = bars;                           // [R]
  uint64_t* kv_full = q_full + R;                    // [R][stages]
  uint64_t* kv_empty = kv_full + R * kStages;        // [R][stages]
  uint64_t* bias_full = kv_empty + R * kStages;      // [stages]
  uint64_t* bias_empty = bias_full + Cfg::kBiasStages;  // [stages]  (one arrival per softmax warp)
  uint64_t* s_full = bias_empty + Cfg::kBiasStages;  // [R][3]
  uint64_t* p_ready = s_full + R * 3;                // [R][3]  (256 arrivals: both streams)
  uint64_t* o_full = p_ready + R * 3;                // [R][3]
  uint64_t* init_ready = o_full + R * 3;             // [R]     (128 arrivals, used once)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(init_ready + R);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qb = blockIdx.x;
  const int h = blockIdx.y;
  const int b0 = blockIdx.z * R;  // first batch entry of this CTA
  // window mode: a query block of 128 atoms = four windows sees the 256 atoms that start 48 before it (two key tiles)
  // Half tiles of 64 keys to process.  Keys after the last valid key of this CTA's pair rows contribute exactly zero
  // (the reference's finite -1e9 underflows in the exponential), so whole half tiles of them are skipped; a row without
  // any valid key keeps the full range (its result is the uniform average over all keys, as in the reference).
  int nhalf = WIN ? 4 : 2 * ((p.lk + kBKV - 1) / kBKV);
  uint32_t* s_last = tmem_slot + 1;                   // [warps]: last valid key + 1 seen by each warp
  constexpr bool kTrim = !WIN && R == 1;
  if (kTrim) {
    const int b_hi = b0 / p.mask_lo_extent, b_lo = b0 - b_hi * p.mask_lo_extent;
    const unsigned char* mrow = p.mask + static_cast<long long>(b_hi) * p.m_hi + static_cast<long long>(b_lo) * p.m_lo;
    int last = 0;
    for (int k = threadIdx.x; k < p.lk; k += blockDim.x)
      if (mrow[static_cast<long long>(k) * p.m_k]) last = k + 1;
    last = __reduce_max_sync(0xffffffffu, last);
    if (lane == 0) s_last[warp] = static_cast<uint32_t>(last);
  }
  long long* trace = (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? p.trace : nullptr;
#ifdef KFB_DEBUG_TRACE
#ifdef KFB_DEBUG_TRACE
#define KFB_STAMP(slot) do { if (trace != nullptr) trace[slot] = clock64(); } while (0)
#else
#define KFB_STAMP(slot) do { (void)trace; } while (0)
#endif
#else
#define KFB_STAMP(slot) do { (void)trace; } while (0)
#endif

  if (threadIdx.x == 0) {
    KFB_STAMP(0);
    ptx::prefetch_tmap(&tm_q);
    ptx::prefetch_tmap(&tm_k);
    ptx::prefetch_tmap(&tm_v);
    ptx::prefetch_tmap(&tm_b);
    for (int g = 0; g < R; ++g) {
      ptx::mbar_init(&q_full[g], 1);
      ptx::mbar_init(&init_ready[g], 128);
      for (int u = 0; u < 3; ++u) {
        ptx::mbar_init(&o_full[g * 3 + u], 1);
        ptx::mbar_init(&s_full[g * 3 + u], 1);
        ptx::mbar_init(&p_ready[g * 3 + u], 256);
      }
      for (int s = 0; s < kStages; ++s) {
        ptx::mbar_init(&kv_full[g * kStages + s], 1);
        ptx::mbar_init(&kv_empty[g * kStages + s], 1);
      }
    }
    for (int s = 0; s < Cfg::kBiasStages; ++s) {
      ptx::mbar_init(&bias_full[s], 1);
      ptx::mbar_init(&bias_empty[s], R * 8);
    }
    ptx::fence_barrier_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  // constant operand e0 (128 x 16, first column ones) and the zero halves of the mask-row operands
  if (warp >= 4 && warp < 8) {
    const int r = (warp - 4) * 32 + lane;
    const uint32_t off = small_operand_row_offset(r);
    // e0: a one in column 0; window mode: a one in column r / 32, the window of query row r (four windows per block)
    const int e_col = WIN ? (r >> 5) : 0;
    *reinterpret_cast<uint4*>(s_e0 + off) = make_uint4(e_col == 0 ? 0x3F80u : (e_col == 1 ? 0x3F800000u : 0u),
                                                      e_col == 2 ? 0x3F80u : (e_col == 3 ? 0x3F800000u : 0u), 0, 0);
    *reinterpret_cast<uint4*>(s_e0 + off + 128) = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < R * 3; ++u)
      *reinterpret_cast<uint4*>(s_maskrow + u * Cfg::kSmallBytes + off + 128) = make_uint4(0, 0, 0, 0);
    ptx::fence_proxy_async_smem();
  }
  // The mask bytes of the first two key tiles (the operands of S(0) .. S(3)) are fetched before the block-wide barrier by
  // the threads that will store them: their latency runs under the tensor-memory allocation and the barrier.
  int early_code0 = 2, early_code1 = 2;
  if (!WIN && warp >= 4 && (((warp - 4) >> 2) & 1) == 0) {
    const int g_ = (warp - 4) >> 3, r_ = (warp & 3) * 32 + lane, b_ = b0 + g_;
    if (b_ < p.batch) {
      const int b_hi = b_ / p.mask_lo_extent, b_lo = b_ - b_hi * p.mask_lo_extent;
      const unsigned char* mrow_ = p.mask + static_cast<long long>(b_hi) * p.m_hi + static_cast<long long>(b_lo) * p.m_lo;
      if (r_ < p.lk) early_code0 = mrow_[static_cast<long long>(r_) * p.m_k] ? 1 : 0;
      if (kBKV + r_ < p.lk) early_code1 = mrow_[static_cast<long long>(kBKV + r_) * p.m_k] ? 1 : 0;
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  bool uniform_row = false;   // no valid key in this pair row: every logit is the same finite -1e9, the result the mean of V
  if (kTrim) {
    uint32_t last = 0;
    for (int wi = 0; wi < Cfg::kThreads / 32; ++wi) last = max(last, s_last[wi]);
    if (last > 0) nhalf = max(2, (static_cast<int>(last) + 63) / 64);
    uniform_row = (last == 0);
  }
  const int nkv = (nhalf + 1) / 2;

  if (uniform_row) {
    // ---------------------------------------------------------------- a pair row without valid keys (padding)
    // The reference adds the same finite -1e9 to every logit of such a row; in float32 the logits then coincide (the
    // spacing of floats at 1e9 is 64) and the softmax is uniform over all lk keys.  The pipeline below computes the same
    // thing with P = 1 everywhere; here the mean of V is taken directly: DPAD rows of V^T, lk keys each.
    float* s_mean = reinterpret_cast<float*>(s_q);                       // [DPAD]
    const __nv_bfloat16* vrows = reinterpret_cast<const __nv_bfloat16*>(p.vt) +
                                 (static_cast<long long>(b0) * p.heads * DPAD + static_cast<long long>(h) * DPAD) * p.ldv;
    for (int dd = warp; dd < DPAD; dd += Cfg::kThreads / 32) {
      const __nv_bfloat162* vr = reinterpret_cast<const __nv_bfloat162*>(vrows + static_cast<long long>(dd) * p.ldv);
      float acc = 0.f;
      for (int k2 = lane; k2 < p.lk / 2; k2 += 32) {
        const float2 f = __bfloat1622float2(vr[k2]);
        acc += f.x + f.y;
      }
      if ((p.lk & 1) && lane == 0) acc += __bfloat162float(vrows[static_cast<long long>(dd) * p.ldv + p.lk - 1]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) s_mean[dd] = acc / static_cast<float>(p.lk);
    }
    __syncthreads();
    if (threadIdx.x < kBQ) {
      const int q_idx = qb * kBQ + threadIdx.x;
      if (q_idx < p.lq) {
        const long long row = static_cast<long long>(b0) * p.lq + q_idx;
        const __nv_bfloat16* gp =
            p.g != nullptr ? reinterpret_cast<const __nv_bfloat16*>(p.g) + row * p.ldg + p.g_col0 + h * DPAD : nullptr;
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.ldo + h * p.d;
        for (int dd = 0; dd < p.d; dd += 8) {   // d is a multiple of 8
          float gs[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) gs[i] = 1.0f;
          if (gp != nullptr) {
            const uint4 gu = *reinterpret_cast<const uint4*>(gp + dd);
            const uint32_t gw[4] = {gu.x, gu.y, gu.z, gu.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              gs[2 * k] = sigmoidf_fast(__uint_as_float(gw[k] << 16));
              gs[2 * k + 1] = sigmoidf_fast(__uint_as_float(gw[k] & 0xffff0000u));
            }
          }
          uint32_t ow[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) ow[k] = pack_bf16x2(s_mean[dd + 2 * k] * gs[2 * k], s_mean[dd + 2 * k + 1] * gs[2 * k + 1]);
          *reinterpret_cast<uint4*>(o + dd) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
      }
    }
  } else

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      for (int g = 0; g < R; ++g) {
        ptx::mbar_expect_tx(&q_full[g], Cfg::kQBytes);
        ptx::tma_load_3d(s_q + g * Cfg::kQBytes, &tm_q, &q_full[g], p.q_col0 + h * DPAD, qb * kBQ, b0 + g);
      }
      const int bias_g = b0 / p.bias_div;
      // window mode: batch entries are samples, bias_mod windows per sample, this block holds windows 4 qb .. 4 qb + 3
      const int bias_b = WIN ? bias_g * p.bias_mod + qb * 4 : (p.bias_mod > 0 ? bias_g * p.bias_mod + b0 % p.bias_mod : bias_g);
      const int bias_z = p.bias_head_major > 0 ? h * p.bias_head_major + bias_b : bias_b * p.heads + h;
      const int bias_zstep = p.bias_head_major > 0 ? 1 : p.heads;   // from one window's bias to the next
      const int key_base = WIN ? qb * kBQ - 48 : 0;               // first key of this block's key range
      bool ok = true;
      int bst = 0;
      uint32_t bpar = 0;   // ring position of the bias half tiles
      for (int j = 0; ok && j < nkv; ++j) {
        const int st = j % kStages;
        for (int g = 0; g < R; ++g) {
          const int slot = g * kStages + st;
          if (!ptx::mbar_wait(&kv_empty[slot], ((j / kStages) & 1) ^ 1, 201)) { ok = false; break; }
          ptx::mbar_expect_tx(&kv_full[slot], Cfg::kKBytes + Cfg::kVBytes);
          // (window mode: rows before atom 0 or past the last atom are outside the tensor and arrive as zeros)
          ptx::tma_load_3d(s_k + slot * Cfg::kKBytes, &tm_k, &kv_full[slot], p.k_col0 + h * DPAD, key_base + j * kBKV, b0 + g);
          ptx::tma_load_3d(s_v + slot * Cfg::kVBytes, &tm_v, &kv_full[slot], key_base + j * kBKV, h * DPAD, b0 + g);
          ptx::tma_load_3d(s_v + slot * Cfg::kVBytes + DPAD * 128, &tm_v, &kv_full[slot], key_base + j * kBKV + 64, h * DPAD, b0 + g);
        }
        for (int hf = 0; ok && hf < 2 && 2 * j + hf < nhalf; ++hf) {
          if (!ptx::mbar_wait(&bias_empty[bst], bpar ^ 1, 202)) { ok = false; break; }
          ptx::mbar_expect_tx(&bias_full[bst], Cfg::kTileBytes);
          if (WIN) {
            // four boxes of 32 rows: window w of the block keeps its bias by window-local key, and its key 0 is key
            // 32 w of the block's range, so the half tile's 64 keys are local keys (j 128 + hf 64 - 32 w) ... + 63; what
            // falls outside [0, 128) arrives as zeros (those keys are masked as absent for that window)
            for (int wq = 0; wq < 4; ++wq)
              ptx::tma_load_3d(s_bias + bst * Cfg::kTileBytes + wq * 4096, &tm_b, &bias_full[bst], j * kBKV + hf * 64 - 32 * wq, 0,
                               bias_z + wq * bias_zstep);
          } else {
            ptx::tma_load_3d(s_bias + bst * Cfg::kTileBytes, &tm_b, &bias_full[bst], j * kBKV + hf * 64, qb * kBQ, bias_z);
          }
          if (++bst == Cfg::kBiasStages) { bst = 0; bpar ^= 1u; }
        }
      }
    }
  } else if (warp <= R) {
    // ---------------------------------------------------------------- MMA issuer of row group g
    // The whole warp runs this loop with warp-uniform values; one elected lane issues the tensor-core instructions.
    {
      const int g = warp - 1;
      const uint32_t tmem_base_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      constexpr uint32_t idesc_s = ptx::make_idesc(kBQ, 64, 1);
      constexpr uint32_t idesc_o = ptx::make_idesc(kBQ, DPAD, 1);
      // operand descriptors are built once; inside the loop only their 16-byte-unit address field advances
      const uint64_t e0_desc = make_noswizzle_desc(ptx::smem_u32(s_e0));
      const uint64_t q_desc = ptx::make_kmajor_desc<Cfg::kSpan>(ptx::smem_u32(s_q + g * Cfg::kQBytes));
      const uint64_t k_desc0 = ptx::make_kmajor_desc<Cfg::kSpan>(ptx::smem_u32(s_k + g * kStages * Cfg::kKBytes));
      const uint64_t v_desc0 = ptx::make_kmajor_desc<128>(ptx::smem_u32(s_v + g * kStages * Cfg::kVBytes));
      const uint64_t m_desc0 = make_noswizzle_desc(ptx::smem_u32(s_maskrow + g * 3 * Cfg::kSmallBytes));
      const uint32_t tmem_s0 = tmem_base_u + g * 192;
      const uint32_t tmem_o0 = tmem_base_u + Cfg::kTmemO + g * 2 * DPAD;
      bool ok = true;

      // S_g(t) = Q_g K_g(t)^T + e0 maskrow_g(t)^T for the 64 keys of half tile t = 2j + hf, into S buffer `buf`;
      // `st` = j % kv stages, `mb` = j % 3 (mask operand buffer)
      auto issue_s = [&](int hf, int buf, int st, uint32_t kv_parity, int mb) -> bool {
        if (hf == 0 && !__all_sync(0xffffffffu, ptx::mbar_wait(&kv_full[g * kStages + st], kv_parity, 204))) return false;
        ptx::tc_fence_after_sync();
        const uint32_t tmem_s = tmem_s0 + buf * 64;
        const uint64_t k_desc = k_desc0 + static_cast<uint32_t>((st * Cfg::kKBytes + hf * 64 * Cfg::kSpan) >> 4);
#pragma unroll
        for (int kk = 0; kk < DPAD / 16; ++kk)
          ptx::mma_f16_ss_warp(tmem_s, q_desc + kk * 2, k_desc + kk * 2, idesc_s, kk != 0 ? 1u : 0u);
        ptx::mma_f16_ss_warp(tmem_s, e0_desc, m_desc0 + static_cast<uint32_t>((mb * Cfg::kSmallBytes + hf * 2048) >> 4), idesc_s, 1u);
        ptx::tc_commit_warp(&s_full[g * 3 + buf]);
        return true;
      };

      ok = __all_sync(0xffffffffu, ptx::mbar_wait(&q_full[g], 0, 205) && ptx::mbar_wait(&init_ready[g], 0, 206)) &&
           issue_s(0, 0, 0, 0, 0) &&
           issue_s(1, 1, 0, 0, 0);
      if (ok && nhalf > 2) ok = issue_s(0, 2, 1 % kStages, (1 / kStages) & 1, 1);
      // half tile t lives in S buffer `buf` = t % 3 (use number `use` = t / 3) and in K/V stage `st` = (t / 2) % 3;
      // half tile t + 3 (issued below) belongs to tile j3 = (t + 3) / 2: stage st3 = j3 % 3, parity par3 = (j3 / 3) & 1
      int buf = 0, st = 0;
      uint32_t use_par = 0;
      int st3 = 1 % kStages, mb3 = 1;             // K/V stage and mask buffer (j3 % 3) of tile j3
      uint32_t par3 = (1 / kStages) & 1;
      for (int t = 0; ok && t < nhalf; ++t) {
        const int hf = t & 1;
        // both streams' P(t) are in tensor memory, the mask rows needed by S(t+3) are written
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&p_ready[g * 3 + buf], use_par, 207))) { ok = false; break; }
        if (lane == 0) KFB_STAMP(16 + (t & 15) * 8 + g * 4 + 1);
        ptx::tc_fence_after_sync();
        const uint64_t v_desc = v_desc0 + static_cast<uint32_t>((st * Cfg::kVBytes + hf * (DPAD * 128)) >> 4);
        const uint32_t tmem_p = tmem_s0 + buf * 64;
        const uint32_t acc_flag = t > 0 ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)  // A = P straight from tensor memory: stream c's 16 columns start at c * 32
          ptx::mma_f16_ts_warp(tmem_o0 + (kk >> 1) * DPAD, tmem_p + (kk >> 1) * 32 + (kk & 1) * 8, v_desc + kk * 2, idesc_o,
                          ((kk & 1) != 0) ? 1u : acc_flag);
        ptx::tc_commit_warp(&o_full[g * 3 + buf]);
        if (hf == 1) ptx::tc_commit_warp(&kv_empty[g * kStages + st]);
        // S(t+3): half (t+3) & 1 = hf ^ 1 of tile j3
        if (t + 3 < nhalf && !issue_s(hf ^ 1, buf, st3, par3, mb3)) { ok = false; break; }
        if (lane == 0) KFB_STAMP(16 + (t & 15) * 8 + g * 4 + 0);
        if (++buf == 3) { buf = 0; use_par ^= 1u; }
        if (hf == 1) { if (++st == kStages) st = 0; }
        // t + 4 belongs to the next tile when t + 4 is even
        if (hf == 0) {
          if (++mb3 == 3) mb3 = 0;
          if (++st3 == kStages) { st3 = 0; par3 ^= 1u; }
        }
      }
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- softmax streams
    const int w = warp - 4;
    const int g = w >> 3;                   // row group
    const int u = (w >> 2) & 1;             // stream: key columns u*32 .. u*32+31 of every half tile
    const int quad = warp & 3;              // TMEM lane quadrant of this warp
    const int r = quad * 32 + lane;         // row inside the query block == TMEM lane
    const int q_idx = qb * kBQ + r;
    const int b = b0 + g;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tmem_s0 = tmem_base + g * 192 + u * 32 + lane_base;
    const uint32_t tmem_o = tmem_base + Cfg::kTmemO + (g * 2 + u) * DPAD + lane_base;
    const int b_hi = b / p.mask_lo_extent, b_lo = b - b_hi * p.mask_lo_extent;
    const unsigned char* mrow = p.mask + static_cast<long long>(b_hi) * p.m_hi + static_cast<long long>(b_lo) * p.m_lo;
    uint8_t* my_maskrow = s_maskrow + g * 3 * Cfg::kSmallBytes + small_operand_row_offset(r);
    const uint8_t* my_bias = s_bias + r * 128;
    const int swz = r & 7;

    // stream 0 provides the mask operand: this thread writes key j*128 + r of tile j
    // code of a key: 0 masked (the reference's finite -1e9), 1 valid, 2 absent.  Window mode returns four codes, two
    // bits each, one per window of the block: key `key` of the block's range is atom key_base + key; window w sees it
    // as its local key (key - 32 w) when that lies in [0, 128), atoms outside the molecule count as masked there.
    auto load_mask_byte = [&](int j) -> int {
      const int key = j * kBKV + r;
      if (WIN) {
        const int atom = qb * kBQ - 48 + key;
        const int in_band = (atom >= 0 && atom < p.lk && mrow[static_cast<long long>(atom) * p.m_k]) ? 1 : 0;
        int code = 0;
#pragma unroll
        for (int wq = 0; wq < 4; ++wq) code |= ((key >= 32 * wq && key < 32 * wq + kBKV) ? in_band : 2) << (2 * wq);
        return code;
      }
      if (key >= p.lk) return 2;
      return mrow[static_cast<long long>(key) * p.m_k] ? 1 : 0;
    };
    auto mask_bits = [](int code) -> uint32_t {
      const float mv = code == 2 ? kAbsent : (code == 1 ? 0.f : kMasked);
      return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(mv)));
    };
    auto store_mask_value = [&](int buf, int code) {
      uint4 v = make_uint4(mask_bits(code & 3), 0, 0, 0);
      if (WIN) {
        v.x |= mask_bits((code >> 2) & 3) << 16;
        v.y = mask_bits((code >> 4) & 3) | (mask_bits((code >> 6) & 3) << 16);
      }
      *reinterpret_cast<uint4*>(my_maskrow + buf * Cfg::kSmallBytes) = v;
    };
    if (u == 0) {
      store_mask_value(0, WIN ? load_mask_byte(0) : early_code0);
      if (nkv > 1) store_mask_value(1, WIN ? load_mask_byte(1) : early_code1);
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(&init_ready[g]);
    }

    float s_cur = 0.f, l_run = 0.f;
    bool ok = true;
    int buf = 0, mbuf = 2;        // S buffer of half tile t (t % 3); mask buffer of tile t/2 + 2
    uint32_t use_par = 0;
    static_assert(Cfg::kBiasStages == 3, "the bias ring is indexed like the S buffers: half tile t sits in stage t % 3");

#pragma unroll 1
    for (int t = 0; t < nhalf; ++t) {
      const int j = t >> 1, hf = t & 1;
      // the mask byte of the next tile is fetched now and used at the end of the pass: its latency hides behind the pass
      int mask_next = 0;
      if (u == 0 && hf == 0 && j + 2 < nkv) mask_next = load_mask_byte(j + 2);
      // (waits of the softmax warps are made warp-uniform: the lanes meet again at the warp-level barriers below)
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&s_full[g * 3 + buf], use_par, 208))) { ok = false; break; }
      if (r == 0) KFB_STAMP(256 + (g * 2 + u) * 64 + (t & 7) * 8 + 0);
      ptx::tc_fence_after_sync();
      float x[32];
      const uint32_t tmem_s = tmem_s0 + buf * 64;
      ptx::tmem_ld_32x32b_x32(tmem_s, reinterpret_cast<uint32_t(&)[32]>(x));
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bias_full[buf], use_par, 203))) { ok = false; break; }
      // the thread's own 64 bytes of its 128-byte row of the bias half tile (16-byte chunks swizzled by the row index)
      const uint8_t* brow = my_bias + buf * Cfg::kTileBytes;
      uint4 bw[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) bw[c] = *reinterpret_cast<const uint4*>(brow + (((u * 4 + c) ^ swz) << 4));
      __syncwarp();  // this warp has read its part of the bias half tile
      if (lane == 0) ptx::mbar_arrive(&bias_empty[buf]);
      ptx::tmem_ld_wait();
      // x = S + log2(e) * bias
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t wv[4] = {bw[c].x, bw[c].y, bw[c].z, bw[c].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          x[c * 8 + q * 2] = fmaf(__uint_as_float(wv[q] << 16), kLog2e, x[c * 8 + q * 2]);
          x[c * 8 + q * 2 + 1] = fmaf(__uint_as_float(wv[q] & 0xffff0000u), kLog2e, x[c * 8 + q * 2 + 1]);
        }
      }
      auto row_max = [&]() -> float {
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          m4[0] = fmaxf(m4[0], x[i]);
          m4[1] = fmaxf(m4[1], x[i + 1]);
          m4[2] = fmaxf(m4[2], x[i + 2]);
          m4[3] = fmaxf(m4[3], x[i + 3]);
        }
        return fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      };
      // P = exp2(x - s) over the first 16 of this stream's own 32 S columns (all of x is in registers); returns the row sum
      const uint32_t tmem_s_w = tmem_s;
      auto exp_pass = [&](float s) -> float {
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t out[8];
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float p0 = exp2f(x[c * 16 + i] - s);
            const float p1 = exp2f(x[c * 16 + i + 1] - s);
            l4[i & 3] += p0;
            l4[(i + 1) & 3] += p1;
            out[i >> 1] = pack_bf16x2(p0, p1);
          }
          ptx::tmem_st_32x32b_x8(tmem_s_w + c * 8, out);
        }
        return (l4[0] + l4[1]) + (l4[2] + l4[3]);
      };
      // The stabiliser s lags: it is the row maximum of the stream's first half tile and is raised only when a half
      // tile's exponentials threaten to overflow (row sum above 2^100: some logit exceeds s by about 95 in log2
      // units).  Any s gives the same result as long as P, the row sum and the accumulator use the same one; the
      // common path therefore needs no row maximum at all.
      float s_use = s_cur;
      if (t == 0) s_use = row_max();
      if (r == 0) KFB_STAMP(256 + (g * 2 + u) * 64 + (t & 7) * 8 + 1);
      float l_blk = exp_pass(s_use);
      if (t > 0 && __any_sync(0xffffffffu, !(l_blk < kRedoSum))) {
        // rare: redo this half tile against its own maximum and move the stream's accumulator and row sum to it,
        // once the P V product issued after the previous pass has completed
        // (o_full[buf] completes one phase per three half tiles: S(t) complete implies P V(t-3) and everything before
        // it complete, and P V(t+2) cannot be issued before this pass and the next two end, so the barrier of
        // half tile t-1 is exactly in the phase waited for: the parity test is unambiguous)
        if (!__all_sync(0xffffffffu,
                        ptx::mbar_wait(&o_full[g * 3 + (buf == 0 ? 2 : buf - 1)], buf == 0 ? (use_par ^ 1u) : use_par, 209))) {
          ok = false;
          break;
        }
        ptx::tc_fence_after_sync();
        if (!(l_blk < kRedoSum)) s_use = fmaxf(row_max(), s_cur);
        const float alpha = exp2f(s_cur - s_use);  // 1 for the lanes whose stabiliser stays
#pragma unroll
        for (int cb = 0; cb < DPAD / 16; ++cb) {
          uint32_t o16[16];
          ptx::tmem_ld_32x32b_x16(tmem_o + cb * 16, o16);
          ptx::tmem_ld_wait();
          uint32_t lo[8], hi[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            lo[i] = __float_as_uint(__uint_as_float(o16[i]) * alpha);
            hi[i] = __float_as_uint(__uint_as_float(o16[8 + i]) * alpha);
          }
          ptx::tmem_st_32x32b_x8(tmem_o + cb * 16, lo);
          ptx::tmem_st_32x32b_x8(tmem_o + cb * 16 + 8, hi);
        }
        l_run *= alpha;
        l_blk = exp_pass(s_use);
      }
      l_run += l_blk;
      s_cur = s_use;
      if (r == 0) KFB_STAMP(256 + (g * 2 + u) * 64 + (t & 7) * 8 + 2);
      if (u == 0 && hf == 0 && j + 2 < nkv) {
        // S(2j) is complete, so every earlier S is too: the mask operand buffer of tile j+2 (last read by tile j-1)
        // is free.  Its first reader, S(2j+4), is issued after the p_ready arrival of half tile 2j+1.
        store_mask_value(mbuf, mask_next);
        ptx::fence_proxy_async_smem();
      }
      if (hf == 0 && ++mbuf == 3) mbuf = 0;
      ptx::tmem_st_wait();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&p_ready[g * 3 + buf]);
      if (++buf == 3) { buf = 0; use_par ^= 1u; }
      if (r == 0) KFB_STAMP(256 + (g * 2 + u) * 64 + (t & 7) * 8 + 3);
    }

    // ---- merge the two streams of the row group and write the result
    // The K stages of this row group are free once both streams have seen their last P V product.
    float* xchg = reinterpret_cast<float*>(s_k + g * kStages * Cfg::kKBytes) + r * Cfg::kXchgStride;
    // (with one row group per CTA the V stages follow the K stages directly and are just as free)
    static_assert(128 * (DPAD + 3) * 4 <= (R == 1 ? kStages * (Cfg::kKBytes + Cfg::kVBytes) : kStages * Cfg::kKBytes),
                  "exchange area does not fit in the K (and V) stages");
    // the gate logits of this row are fetched now, under the wait for the last product and the exchange of the streams
    const bool row_ok = q_idx < p.lq;  // rows past the end still take part in the warp-wide loads
    const long long row = static_cast<long long>(b) * p.lq + (row_ok ? q_idx : 0);
    const __nv_bfloat16* gp =
        p.g != nullptr ? reinterpret_cast<const __nv_bfloat16*>(p.g) + row * p.ldg + p.g_col0 + h * DPAD : nullptr;
    uint4 gate_raw[DPAD / 8];
    if (u == 0 && gp != nullptr) {
#pragma unroll
      for (int i = 0; i < DPAD / 8; ++i) gate_raw[i] = *reinterpret_cast<const uint4*>(gp + i * 8);
    }
    // the last P V product: then all of them are complete
    ok = ok && ptx::mbar_wait(&o_full[g * 3 + (nhalf - 1) % 3], ((nhalf - 1) / 3) & 1, 210);
    ok = __all_sync(0xffffffffu, ok);  // the tensor-memory loads below are warp-wide: decide per warp
    if (u == 1) {
      if (ok) {
        ptx::tc_fence_after_sync();
#pragma unroll
        for (int cb = 0; cb < DPAD / 16; ++cb) {
          uint32_t o16[16];
          ptx::tmem_ld_32x32b_x16(tmem_o + cb * 16, o16);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) xchg[cb * 16 + i] = __uint_as_float(o16[i]);
        }
        xchg[DPAD] = s_cur;
        xchg[DPAD + 1] = l_run;
      } else {
        xchg[DPAD + 1] = -1.f;  // tells the partner that this stream gave up
      }
    }
    // all 8 warps of the row group meet here exactly once, whatever happened above
    asm volatile("bar.sync %0, 256;" ::"r"(1 + g) : "memory");
    if (u == 0 && __all_sync(0xffffffffu, ok && xchg[DPAD + 1] >= 0.f)) {
      ptx::tc_fence_after_sync();
      const float s_o = xchg[DPAD], l_o = xchg[DPAD + 1];
      const float s_m = fmaxf(s_cur, s_o);
      const float w_e = exp2f(s_cur - s_m), w_o = exp2f(s_o - s_m);
      const float inv_l = 1.0f / (l_run * w_e + l_o * w_o);
      const float c_e = w_e * inv_l, c_o = w_o * inv_l;
      __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.ldo + h * p.d;
      {
#pragma unroll
        for (int cb = 0; cb < DPAD / 16; ++cb) {
          uint32_t o16[16];
          ptx::tmem_ld_32x32b_x16(tmem_o + cb * 16, o16);
          ptx::tmem_ld_wait();
          float v[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(o16[i]) * c_e + xchg[cb * 16 + i] * c_o;
          if (gp != nullptr) {
#pragma unroll
            for (int i = 0; i < 16; i += 8) {
              const uint4 gu = gate_raw[cb * 2 + i / 8];
              const uint32_t gw[4] = {gu.x, gu.y, gu.z, gu.w};
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                v[i + k * 2] *= sigmoidf_fast(__uint_as_float(gw[k] << 16));
                v[i + k * 2 + 1] *= sigmoidf_fast(__uint_as_float(gw[k] & 0xffff0000u));
              }
            }
          }
          uint32_t ow[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) ow[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
          if (row_ok && cb * 16 + 16 <= p.d && (reinterpret_cast<uintptr_t>(o + cb * 16) & 31) == 0) {
            // 32-byte store: one full sector per instruction
            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(o + cb * 16), "r"(ow[0]), "r"(ow[1]),
                         "r"(ow[2]), "r"(ow[3]), "r"(ow[4]), "r"(ow[5]), "r"(ow[6]), "r"(ow[7])
                         : "memory");
          } else {
#pragma unroll
            for (int i = 0; i < 16; i += 8) {
              if (row_ok && cb * 16 + i < p.d)  // d is a multiple of 8
                *reinterpret_cast<uint4*>(o + cb * 16 + i) = make_uint4(ow[i / 2], ow[i / 2 + 1], ow[i / 2 + 2], ow[i / 2 + 3]);
            }
          }
        }
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) KFB_STAMP(1);
#undef KFB_STAMP
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

static long long* g_attention_trace = nullptr;
void set_attention_trace(long long* device_buffer) { g_attention_trace = device_buffer; }

template <int DPAD, int R, bool WIN = false>
static int launch_cfg(cudaStream_t stream, const AttnParams& p) {
  using Cfg = AttCfg<DPAD, R>;
  static std::once_flag once[64];
  int dev = 0;
  KFB_CUDA(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  std::call_once(once[dev & 63], [&] {
    attr_err = cudaFuncSetAttribute(attention_bias_kernel<DPAD, R, WIN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::kSmemBytes);
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
    const int bias_batches = p.bias_head_major > 0 ? p.bias_head_major : cdiv(p.batch, p.bias_div) * (p.bias_mod > 0 ? p.bias_mod : 1);
    if (p.win) {
      // one bias per window: [z][32 queries][128 local keys], fetched in boxes of 32 rows
      const uint64_t dims[3] = {128, 32, (uint64_t)bias_batches * p.heads};
      const uint64_t str[2] = {128 * 2, 32 * 128 * 2};
      const uint32_t box[3] = {64, 32, 1};
      KFB_TRY(make_tmap(&tb, p.bias, 2, 3, dims, str, box, 128));
    } else {
      const uint64_t dims[3] = {(uint64_t)p.lk, (uint64_t)p.lq, (uint64_t)bias_batches * p.heads};
      const uint64_t str[2] = {(uint64_t)p.ldb * 2, (uint64_t)p.lq * p.ldb * 2};
      const uint32_t box[3] = {64, kBQ, 1};
      KFB_TRY(make_tmap(&tb, p.bias, 2, 3, dims, str, box, 128));
    }
  }
  dim3 grid(cdiv(p.lq, kBQ), p.heads, p.batch / R);
  {
    LaunchScope scope(stream, p.tag ? p.tag : "attention");
    attention_bias_kernel<DPAD, R, WIN><<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(tq, tk, tv, tb, p);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

int launch_attention(cudaStream_t stream, const AttnParams& p_in) {
  AttnParams p = p_in;
  p.trace = g_attention_trace;
  KFB_CHECK_ARG(p.batch > 0 && p.heads > 0 && p.lq > 0 && p.lk > 0, "attention: empty problem");
  KFB_CHECK_ARG(p.d % 8 == 0 && p.d <= p.dpad, "attention: head dim %d must be a multiple of 8 and <= %d", p.d, p.dpad);
  KFB_CHECK_ARG(p.ldq % 8 == 0 && p.ldk % 8 == 0 && p.ldv % 8 == 0 && p.ldb % 8 == 0 && p.ldo % 8 == 0,
                "attention: leading dimensions must be multiples of 8 elements");
  KFB_CHECK_ARG(p.bias_div >= 1 && p.bias_mod >= 0 && p.mask_lo_extent >= 1, "attention: bad divisors");
  KFB_CHECK_ARG(p.bias_head_major == 0 || p.bias_head_major >= cdiv(p.batch, p.bias_div) * (p.bias_mod > 0 ? p.bias_mod : 1),
                "attention: head-major bias with %d batches is too small", p.bias_head_major);
  KFB_CHECK_ARG(p.batch <= 65535, "attention: batch %d exceeds the grid z limit", p.batch);
  if (p.win) {
    KFB_CHECK_ARG(p.dpad == 32 && p.lq == p.lk && p.lq % 32 == 0 && p.bias_mod == p.lq / 32,
                  "attention: window mode needs head dim <= 32, Lq == Lk a multiple of 32 and bias_mod == Lq / 32 windows");
    return launch_cfg<32, 1, true>(stream, p);
  }
  // head dim <= 32: one row group per CTA, two CTAs resident per SM -- they interleave their softmax and tensor-core
  // phases better than two row groups inside one CTA did (measured 6 % faster at N=768); the bias tile both read stays
  // in L2
  if (p.dpad == 32) return launch_cfg<32, 1>(stream, p);
  if (p.dpad == 64) return launch_cfg<64, 1>(stream, p);
  set_error("attention: padded head dim %d not supported (32 or 64)", p.dpad);
  return KFB_ERR_UNSUPPORTED;
}

}  // namespace kfb
