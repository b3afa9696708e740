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
static constexpr float kMasked = -1e9f;         // additive value of a masked key (finite, as in the reference)
static constexpr float kAbsent = -1e30f;        // keys beyond lk
static constexpr float kRaiseThreshold = 5.5f;  // raise the stabiliser when the running max moved by more than e^5.5
static constexpr float kRedoThreshold = 60.f;   // redo a block whose exponents would approach fp32 overflow

template <int DPAD, int R>
struct AttCfg {
  static constexpr int kThreads = 64 + 128 * R;
  static constexpr int kSpan = DPAD * 2;                 // bytes per q/k row = swizzle span
  static constexpr int kQBytes = kBQ * kSpan;            // per row group
  static constexpr int kKBytes = kBKV * kSpan;
  static constexpr int kVBytes = 2 * DPAD * 128;         // two boxes of [DPAD rows x 64 keys]
  static constexpr int kKvStages = 2;
  static constexpr int kTileBytes = 2 * 128 * 128;       // a 128 x 128 bf16 tile as two 64-wide swizzled halves
  static constexpr int kSmallBytes = 128 * 32;           // a 128 x 16 bf16 K-major operand without swizzle
  static constexpr int kBiasStages = 2;
  // tensor memory columns: S_g at g*128 (fp32), O_g at R*128 + g*DPAD (fp32), P_g at R*(128+DPAD) + g*64 (bf16 pairs),
  // then the constant identity matrix
  static constexpr int kTmemO = R * 128;
  static constexpr int kTmemP = R * (128 + DPAD);
  static constexpr int kTmemI = R * (128 + DPAD + 64);   // identity (128 x 128 bf16 = 64 columns), A operand of the bias MMA
  static constexpr int kTmemCols = (kTmemI + 64 <= 256) ? 256 : 512;
  static constexpr int kSmemBytes = R * kQBytes + R * kKvStages * (kKBytes + kVBytes) + kBiasStages * kTileBytes /*bias*/ +
                                    kSmallBytes /*e0*/ +
                                    R * kSmallBytes /*mask rows*/ + 1024 /*align*/ + 256 /*barriers*/;
};

// K-major operand without swizzle: 8 x 8 core matrices (8 rows of 16 bytes); the two K halves of a K=16
// slice are 128 bytes apart (leading byte offset), groups of 8 rows 256 bytes apart (stride byte offset).
__device__ __forceinline__ uint64_t make_noswizzle_desc(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4) | (static_cast<uint64_t>(128 >> 4) << 16) |
         (static_cast<uint64_t>(256 >> 4) << 32) | (1ull << 46);
}
// MN-major operand tile made of 128-byte swizzled rows: row = one K index holding 64 contiguous MN elements
// (what a TMA box of 64 x rows with 128B swizzle writes).  Groups of 8 K-rows are 1024 bytes apart (stride
// byte offset); the next 64 MN elements live in the next box, `mn_group_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t make_mnmajor_desc(uint32_t smem_addr, uint32_t mn_group_bytes) {
  return static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4) | (static_cast<uint64_t>(mn_group_bytes >> 4) << 16) |
         (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint32_t small_operand_row_offset(int r) { return (r >> 3) * 256 + (r & 7) * 16; }

template <int DPAD, int R>
__global__ void __launch_bounds__(AttCfg<DPAD, R>::kThreads) __maxnreg__((R == 1) ? 255 : 168)
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
  uint8_t* s_bias = s_v + R * kStages * Cfg::kVBytes;
  uint8_t* s_e0 = s_bias + Cfg::kBiasStages * Cfg::kTileBytes;
  uint8_t* s_maskrow = s_e0 + Cfg::kSmallBytes;                   // [R]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_maskrow + R * Cfg::kSmallBytes);
  uint64_t* q_full = bars;                           // [R]
  uint64_t* kv_full = q_full + R;                    // [R][stages]
  uint64_t* kv_empty = kv_full + R * kStages;        // [R][stages]
  uint64_t* bias_full = kv_empty + R * kStages;
  uint64_t* bias_empty = bias_full + Cfg::kBiasStages;
  uint64_t* s_full = bias_empty + Cfg::kBiasStages;  // [R]
  uint64_t* ready = s_full + R;                      // [R]  (128 arrivals)
  uint64_t* o_full = ready + R;                      // [R]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + R);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qb = blockIdx.x;
  const int h = blockIdx.y;
  const int b0 = blockIdx.z * R;  // first batch entry of this CTA
  const int nkv = (p.lk + kBKV - 1) / kBKV;
  long long* trace = (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? p.trace : nullptr;
#define KFB_STAMP(slot) do { if (trace != nullptr) trace[slot] = clock64(); } while (0)

  if (threadIdx.x == 0) {
    KFB_STAMP(0);
    ptx::prefetch_tmap(&tm_q);
    ptx::prefetch_tmap(&tm_k);
    ptx::prefetch_tmap(&tm_v);
    ptx::prefetch_tmap(&tm_b);
    for (int g = 0; g < R; ++g) {
      ptx::mbar_init(&q_full[g], 1);
      ptx::mbar_init(&s_full[g], 1);
      ptx::mbar_init(&ready[g], 128);
      ptx::mbar_init(&o_full[g], 1);
      for (int s = 0; s < kStages; ++s) {
        ptx::mbar_init(&kv_full[g * kStages + s], 1);
        ptx::mbar_init(&kv_empty[g * kStages + s], 1);
      }
    }
    for (int s = 0; s < Cfg::kBiasStages; ++s) {
      ptx::mbar_init(&bias_full[s], 1);
      ptx::mbar_init(&bias_empty[s], 1);
    }
    ptx::fence_barrier_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  // constant operand e0 (128 x 16, first column ones) and the zero halves of the mask-row operands
  if (warp >= 2 && warp < 6) {
    const int r = (warp - 2) * 32 + lane;
    const uint32_t off = small_operand_row_offset(r);
    *reinterpret_cast<uint4*>(s_e0 + off) = make_uint4(0x3F80u, 0, 0, 0);
    *reinterpret_cast<uint4*>(s_e0 + off + 128) = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int g = 0; g < R; ++g)
      *reinterpret_cast<uint4*>(s_maskrow + g * Cfg::kSmallBytes + off + 128) = make_uint4(0, 0, 0, 0);
    ptx::fence_proxy_async_smem();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // the identity matrix in tensor memory: row r holds a single bf16 1.0 at K index r (column r/2, half r&1)
  if (warp >= 2 && warp < 6) {
    const int r = (warp & 3) * 32 + lane;
    const uint32_t base = tmem_base + Cfg::kTmemI + (static_cast<uint32_t>((warp & 3) * 32) << 16);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint32_t v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = (c * 8 + i == (r >> 1)) ? (0x3F80u << (16 * (r & 1))) : 0u;
      ptx::tmem_st_32x32b_x8(base + c * 8, v);
    }
    ptx::tmem_st_wait();
    ptx::tc_fence_before_sync();
  }
  __syncthreads();
  ptx::tc_fence_after_sync();

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      for (int g = 0; g < R; ++g) {
        ptx::mbar_expect_tx(&q_full[g], Cfg::kQBytes);
        ptx::tma_load_3d(s_q + g * Cfg::kQBytes, &tm_q, &q_full[g], p.q_col0 + h * DPAD, qb * kBQ, b0 + g);
      }
      const int bias_z = (b0 / p.bias_div) * p.heads + h;
      bool ok = true;
      for (int j = 0; ok && j < nkv; ++j) {
        const int bs = j % Cfg::kBiasStages;
        if (!ptx::mbar_wait(&bias_empty[bs], ((j / Cfg::kBiasStages) & 1) ^ 1, 202)) break;
        ptx::mbar_expect_tx(&bias_full[bs], Cfg::kTileBytes);
        ptx::tma_load_3d(s_bias + bs * Cfg::kTileBytes, &tm_b, &bias_full[bs], j * kBKV, qb * kBQ, bias_z);
        ptx::tma_load_3d(s_bias + bs * Cfg::kTileBytes + 16384, &tm_b, &bias_full[bs], j * kBKV + 64, qb * kBQ, bias_z);
        const int st = j % kStages;
        for (int g = 0; g < R; ++g) {
          const int slot = g * kStages + st;
          if (!ptx::mbar_wait(&kv_empty[slot], ((j / kStages) & 1) ^ 1, 201)) { ok = false; break; }
          ptx::mbar_expect_tx(&kv_full[slot], Cfg::kKBytes + Cfg::kVBytes);
          ptx::tma_load_3d(s_k + slot * Cfg::kKBytes, &tm_k, &kv_full[slot], p.k_col0 + h * DPAD, j * kBKV, b0 + g);
          ptx::tma_load_3d(s_v + slot * Cfg::kVBytes, &tm_v, &kv_full[slot], j * kBKV, h * DPAD, b0 + g);
          ptx::tma_load_3d(s_v + slot * Cfg::kVBytes + DPAD * 128, &tm_v, &kv_full[slot], j * kBKV + 64, h * DPAD, b0 + g);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = ptx::make_idesc(kBQ, kBKV, 1);
      constexpr uint32_t idesc_o = ptx::make_idesc(kBQ, DPAD, 1);
      constexpr uint32_t idesc_s_bmn = idesc_s | (1u << 16);  // B operand MN-major (the bias tile as it lies in memory)
      const uint64_t e0_desc = make_noswizzle_desc(ptx::smem_u32(s_e0));
      uint64_t maskrow_desc[R];
#pragma unroll
      for (int g = 0; g < R; ++g) maskrow_desc[g] = make_noswizzle_desc(ptx::smem_u32(s_maskrow + g * Cfg::kSmallBytes));
      const uint64_t bias_desc0 = make_mnmajor_desc(ptx::smem_u32(s_bias), 16384);
      const uint32_t tmem_ident = tmem_base + Cfg::kTmemI;
      bool ok = true;

      // S_g(j) = Q_g K_g(j)^T + I bias(j) + e0 maskrow_g(j)^T
      auto issue_s = [&](int g, int j) -> bool {
        const int slot = g * kStages + (j % kStages);
        const int bs = j % Cfg::kBiasStages;
        if (!ptx::mbar_wait(&kv_full[slot], (j / kStages) & 1, 204)) return false;
        if (g == 0 && !ptx::mbar_wait(&bias_full[bs], (j / Cfg::kBiasStages) & 1, 203)) return false;
        ptx::tc_fence_after_sync();
        // descriptors are built once per tile; inside a tile only the 16-byte-unit address field advances, so
        // the single issuing thread spends a couple of instructions per MMA rather than a dependent chain
        const uint32_t tmem_s = tmem_base + g * 128;
        const uint64_t q_desc = ptx::make_kmajor_desc<Cfg::kSpan>(ptx::smem_u32(s_q + g * Cfg::kQBytes));
        const uint64_t k_desc = ptx::make_kmajor_desc<Cfg::kSpan>(ptx::smem_u32(s_k + slot * Cfg::kKBytes));
#pragma unroll
        for (int kk = 0; kk < DPAD / 16; ++kk)
          ptx::mma_f16_ss(tmem_s, q_desc + kk * 2, k_desc + kk * 2, idesc_s, kk != 0 ? 1u : 0u);
        ptx::mma_f16_ss(tmem_s, e0_desc, maskrow_desc[g], idesc_s, 1u);
        // identity (from tensor memory) x bias tile (MN-major, as it lies in memory): the otherwise idle tensor
        // core adds the pair bias; K runs over the 128 queries of the tile, 16 per step
        const uint64_t bias_desc = bias_desc0 + static_cast<uint64_t>(bs) * (Cfg::kTileBytes >> 4);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          ptx::mma_f16_ts(tmem_s, tmem_ident + kk * 8, bias_desc + kk * (2048 >> 4), idesc_s_bmn, 1u);
        ptx::tc_commit(&s_full[g]);
        if (g == R - 1) ptx::tc_commit(&bias_empty[bs]);
        KFB_STAMP(16 + j * 8 + g * 4 + 0);
        return true;
      };

      for (int g = 0; ok && g < R; ++g) {
        ok = ptx::mbar_wait(&q_full[g], 0, 205) && ptx::mbar_wait(&ready[g], 0, 206) && issue_s(g, 0);
      }
      for (int j = 0; ok && j < nkv; ++j) {
        for (int g = 0; ok && g < R; ++g) {
          // P_g(j) is in tensor memory, S_g(j) consumed, O_g(j-1) folded, mask row of block j+1 written
          if (!ptx::mbar_wait(&ready[g], (j + 1) & 1, 207)) { ok = false; break; }
          KFB_STAMP(16 + j * 8 + g * 4 + 1);
          ptx::tc_fence_after_sync();
          // the next S first: it is short and lets the group's next softmax pass start while P V runs
          if (j + 1 < nkv && !issue_s(g, j + 1)) { ok = false; break; }
          const int slot = g * kStages + (j % kStages);
          const uint64_t v_desc = ptx::make_kmajor_desc<128>(ptx::smem_u32(s_v + slot * Cfg::kVBytes));
          const uint32_t tmem_o = tmem_base + Cfg::kTmemO + g * DPAD;
          const uint32_t tmem_p = tmem_base + Cfg::kTmemP + g * 64;
#pragma unroll
          for (int kk = 0; kk < kBKV / 16; ++kk)  // A = P straight from tensor memory, 8 columns per K=16 slice
            ptx::mma_f16_ts(tmem_o, tmem_p + kk * 8, v_desc + ((kk >> 2) * (DPAD * 128 >> 4) + (kk & 3) * 2), idesc_o,
                            kk != 0 ? 1u : 0u);
          ptx::tc_commit(&o_full[g]);
          ptx::tc_commit(&kv_empty[slot]);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + accumulation
    const int g = (warp - 2) >> 2;          // row group
    const int quad = warp & 3;              // TMEM lane quadrant of this warp
    const int r = quad * 32 + lane;         // row inside the query block == TMEM lane
    const int q_idx = qb * kBQ + r;
    const int b = b0 + g;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tmem_s = tmem_base + g * 128 + lane_base;
    const uint32_t tmem_o = tmem_base + Cfg::kTmemO + g * DPAD + lane_base;
    const uint32_t tmem_p = tmem_base + Cfg::kTmemP + g * 64 + lane_base;
    const int b_hi = b / p.mask_lo_extent, b_lo = b - b_hi * p.mask_lo_extent;
    const unsigned char* mrow = p.mask + static_cast<long long>(b_hi) * p.m_hi + static_cast<long long>(b_lo) * p.m_lo;
    uint8_t* my_maskrow = s_maskrow + g * Cfg::kSmallBytes + small_operand_row_offset(r);

    // this thread provides key j*128 + r of its group's mask operand
    auto load_mask_value = [&](int j) -> float {
      const int key = j * kBKV + r;
      if (key >= p.lk) return kAbsent;
      return mrow[static_cast<long long>(key) * p.m_k] ? 0.f : kMasked;
    };
    auto store_mask_value = [&](float mv) {
      const uint32_t bits = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(mv)));
      *reinterpret_cast<uint4*>(my_maskrow) = make_uint4(bits, 0, 0, 0);
    };

    store_mask_value(load_mask_value(0));
    ptx::fence_proxy_async_smem();
    ptx::mbar_arrive(&ready[g]);

    float acc[DPAD];
#pragma unroll
    for (int i = 0; i < DPAD; ++i) acc[i] = 0.f;
    float s_cur = 0.f, l_run = 0.f, s_next = 0.f;
    bool ok = true;

    for (int j = 0; j < nkv; ++j) {
      // the mask byte of the next block is fetched before the wait so that its latency hides behind it
      const float mask_next = (j + 1 < nkv) ? load_mask_value(j + 1) : 0.f;
      if (!ptx::mbar_wait(&s_full[g], j & 1, 208)) { ok = false; break; }
      if (r == 0) KFB_STAMP(256 + g * 128 + j * 8 + 0);
      ptx::tc_fence_after_sync();
      if (j + 1 < nkv) store_mask_value(mask_next);  // S(j) is complete, the MMA no longer reads the mask operand

      if (j == 0) {  // stabiliser of the first block: its true row maximum
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        uint32_t raw0[16], raw1[16];
        ptx::tmem_ld_32x32b_x16(tmem_s, raw0);
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
          ptx::tmem_ld_wait();
          ptx::tmem_ld_32x32b_x16(tmem_s + cc * 32 + 16, raw1);
#pragma unroll
          for (int i = 0; i < 16; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(raw0[i]));
          ptx::tmem_ld_wait();
          if (cc < 3) ptx::tmem_ld_32x32b_x16(tmem_s + cc * 32 + 32, raw0);
#pragma unroll
          for (int i = 0; i < 16; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(raw1[i]));
        }
        s_next = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        s_cur = s_next;
      }

      // single pass: P = exp(S - s_use) = exp2(S * log2e - s_use * log2e).  The first quarter of P
      // waits in registers (packed bf16) until the previous block's P V product has finished reading the P
      // columns of tensor memory; by the second half that is long done and P is stored as it is produced.
      float s_use = s_next, l_blk = 0.f, mx = -INFINITY;
      bool folded = (j == 0);
#pragma unroll 1
      for (int attempt = 0; attempt < 2; ++attempt) {
        const float neg_s = -s_use * kLog2e;
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        auto process = [&](const uint32_t (&raw)[16], int c, uint32_t (&out)[8]) {
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float t0 = __uint_as_float(raw[i]);
            const float t1 = __uint_as_float(raw[i + 1]);
            m4[i & 3] = fmaxf(m4[i & 3], t0);
            m4[(i + 1) & 3] = fmaxf(m4[(i + 1) & 3], t1);
            const float p0 = exp2f(fmaf(t0, kLog2e, neg_s));
            const float p1 = exp2f(fmaf(t1, kLog2e, neg_s));
            l4[i & 3] += p0;
            l4[(i + 1) & 3] += p1;
            out[i >> 1] = pack_bf16x2(p0, p1);
          }
        };
        uint32_t raw0[16], raw1[16];
        {
          // keys 0..31: P waits in registers until the previous block's P V product has released the P columns
          uint32_t held0[8], held1[8];
          ptx::tmem_ld_32x32b_x16(tmem_s, raw0);
          ptx::tmem_ld_wait();
          ptx::tmem_ld_32x32b_x16(tmem_s + 16, raw1);
          process(raw0, 0, held0);
          ptx::tmem_ld_wait();
          ptx::tmem_ld_32x32b_x16(tmem_s + 32, raw0);
          process(raw1, 1, held1);
          if (!folded) {
            // fold the previous block's P V product (same scale as acc)
            if (!ptx::mbar_wait(&o_full[g], (j - 1) & 1, 209)) { ok = false; break; }
            ptx::tc_fence_after_sync();
#pragma unroll
            for (int cb = 0; cb < DPAD / 32; ++cb) {
              uint32_t raw[32];
              ptx::tmem_ld_32x32b_x32(tmem_o + cb * 32, raw);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) acc[cb * 32 + i] += __uint_as_float(raw[i]);
            }
            folded = true;
          }
          ptx::tmem_st_32x32b_x8(tmem_p, held0);
          ptx::tmem_st_32x32b_x8(tmem_p + 8, held1);
        }
#pragma unroll 1
        for (int c = 2; c < 8; c += 2) {  // keys 32..127: stored as produced
          uint32_t out[8];
          ptx::tmem_ld_wait();
          ptx::tmem_ld_32x32b_x16(tmem_s + c * 16 + 16, raw1);
          process(raw0, c, out);
          ptx::tmem_st_32x32b_x8(tmem_p + c * 8, out);
          ptx::tmem_ld_wait();
          if (c + 2 < 8) ptx::tmem_ld_32x32b_x16(tmem_s + c * 16 + 32, raw0);
          process(raw1, c + 1, out);
          ptx::tmem_st_32x32b_x8(tmem_p + c * 8 + 8, out);
        }
        l_blk = (l4[0] + l4[1]) + (l4[2] + l4[3]);
        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        if (mx - s_use <= kRedoThreshold) break;
        s_use = mx;  // exponents too large for comfort: redo this block against its own maximum
      }
      if (!ok) break;
      if (r == 0) KFB_STAMP(256 + g * 128 + j * 8 + 1);
      const float alpha = exp2f((s_cur - s_use) * kLog2e);
#pragma unroll
      for (int i = 0; i < DPAD; ++i) acc[i] *= alpha;
      l_run = l_run * alpha + l_blk;
      s_cur = s_use;
      s_next = (mx > s_cur + kRaiseThreshold) ? mx : s_cur;

      if (r == 0) KFB_STAMP(256 + g * 128 + j * 8 + 2);
      ptx::tmem_st_wait();
      ptx::tc_fence_before_sync();
      ptx::fence_proxy_async_smem();  // the mask row of the next block was written through the generic proxy
      ptx::mbar_arrive(&ready[g]);
    }
    if (ok && ptx::mbar_wait(&o_full[g], (nkv - 1) & 1, 210)) {
      ptx::tc_fence_after_sync();
      const float inv_l = 1.0f / l_run;
#pragma unroll
      for (int c = 0; c < DPAD / 32; ++c) {
        uint32_t raw[32];
        ptx::tmem_ld_32x32b_x32(tmem_o + c * 32, raw);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[c * 32 + i] = (acc[c * 32 + i] + __uint_as_float(raw[i])) * inv_l;
      }
      if (q_idx < p.lq) {
        const long long row = static_cast<long long>(b) * p.lq + q_idx;
        if (p.g != nullptr) {
          const __nv_bfloat16* gp = reinterpret_cast<const __nv_bfloat16*>(p.g) + row * p.ldg + p.g_col0 + h * DPAD;
#pragma unroll
          for (int i = 0; i < DPAD; i += 8) {
            const uint4 u = *reinterpret_cast<const uint4*>(gp + i);
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
  if (threadIdx.x == 0) KFB_STAMP(1);
#undef KFB_STAMP
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

static long long* g_attention_trace = nullptr;
void set_attention_trace(long long* device_buffer) { g_attention_trace = device_buffer; }

template <int DPAD, int R>
static int launch_cfg(cudaStream_t stream, const AttnParams& p) {
  using Cfg = AttCfg<DPAD, R>;
  static std::once_flag once[64];
  int dev = 0;
  KFB_CUDA(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  std::call_once(once[dev & 63], [&] {
    attr_err = cudaFuncSetAttribute(attention_bias_kernel<DPAD, R>, cudaFuncAttributeMaxDynamicSharedMemorySize,
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
    const int bias_batches = cdiv(p.batch, p.bias_div);
    const uint64_t dims[3] = {(uint64_t)p.lk, (uint64_t)p.lq, (uint64_t)bias_batches * p.heads};
    const uint64_t str[2] = {(uint64_t)p.ldb * 2, (uint64_t)p.lq * p.ldb * 2};
    const uint32_t box[3] = {64, kBQ, 1};
    KFB_TRY(make_tmap(&tb, p.bias, 2, 3, dims, str, box, 128));
  }
  dim3 grid(cdiv(p.lq, kBQ), p.heads, p.batch / R);
  {
    LaunchScope scope(stream, p.tag ? p.tag : "attention");
    attention_bias_kernel<DPAD, R><<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(tq, tk, tv, tb, p);
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
  KFB_CHECK_ARG(p.bias_div >= 1 && p.mask_lo_extent >= 1, "attention: bad divisors");
  KFB_CHECK_ARG(p.batch <= 65535, "attention: batch %d exceeds the grid z limit", p.batch);
  if (p.dpad == 32) {
    // two batch rows per CTA when consecutive rows share their bias tile
    if (p.batch % 2 == 0 && p.bias_div % 2 == 0) return launch_cfg<32, 2>(stream, p);
    return launch_cfg<32, 1>(stream, p);
  }
  if (p.dpad == 64) return launch_cfg<64, 1>(stream, p);
  set_error("attention: padded head dim %d not supported (32 or 64)", p.dpad);
  return KFB_ERR_UNSUPPORTED;
}

}  // namespace kfb
