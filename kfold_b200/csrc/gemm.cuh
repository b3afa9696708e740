// Persistent, warp-specialised tcgen05 GEMM:  D[row, col] = sum_k A[row, k] * B[col, k]
//
// Both operands are bf16 and K-major in global memory.  One CTA per SM walks a
// static list of 128 x BN output tiles.  Per tile:
//   warp 0 (one lane)  TMA producer: A and B k-blocks (64 wide = one 128-byte swizzle span)
//                      into a ring of shared-memory stages;
//   warp 1 (one lane)  issues tcgen05.mma (M=128, N=BN, K=16) into one of two TMEM
//                      accumulator buffers (2 x BN fp32 columns), so the epilogue of
//                      tile t overlaps the main loop of tile t+1;
//   warps 2..9         epilogue: each thread owns one accumulator row (one TMEM lane) and every
//                      other 32-column chunk of it,
//                      reads it 32 columns at a time with tcgen05.ld and applies the
//                      fused element-wise tail (gated linear unit, row mask, sigmoid
//                      gate from memory, residual) before storing.
//
// Rows of A are addressed as (batch, o, n) with tiles running along n, so the same
// kernel serves flat [M, K] activations, a transposed walk over an (N x N) pair
// tensor (swap the o / n strides in the tensor map), and the batched per-channel
// triangle contraction.  Out-of-range rows/columns/k are zero-filled by TMA and
// the stores are predicated, so no size needs to be a multiple of the tile.
#pragma once
#include <cuda_bf16.h>

#include "ptx.cuh"

namespace kfb {

enum GluMode : int { GLU_NONE = 0, GLU_SIGMOID = 1, GLU_SWIGLU = 2 };

// One segment of output columns.  Element (row=(b,o,n), col) of the segment goes to
//   dst + b*s_b + o*s_o + n*s_n + (col - col_begin)*s_col      (strides in elements)
struct EpiSeg {
  int col_begin;    // first output column of the segment (multiple of 32)
  int ncols;        // valid columns in the segment; columns beyond are dropped
  int out_fp32;     // 0: bf16 output, 1: fp32 output
  int vec;          // 1: s_col == 1 and every row start is 16-byte aligned -> vector stores
  int tma_slot;     // >= 0: channel-major bf16 segment stored through shared memory with TMA store map `tma_slot`
  int split;        // precise mode: 0 plain store; 1 / 2: the value is split into three bf16 parts x0+x1+x2 and stored
                    // six times, s_part elements apart, as [x0 x0 x1 x1 x0 x2] (1) or [x0 x1 x0 x1 x2 x0] (2)
  long long s_part;
  void* dst;
  long long s_col, s_n, s_o, s_b;
};

struct GemmParams {
  int n_extent, o_extent, batch;  // A rows = batch x o_extent x n_extent
  int n_cols;                     // GEMM columns (rows of B) before GLU pairing
  int k_extent;
  int b_batched;                  // B carries the batch dimension too
  int b_col_inner;                // rows of B are addressed as (col / b_col_inner, col % b_col_inner): an all-gathered
                                  // operand whose pieces lie rank after rank (launcher; = n_cols when not split)
  int n_blocks, num_m_tiles, num_n_tiles;
  int step_n_tile, step_nb, step_o, step_b;  // launcher: the grid size as digits of (n tile, row block, outer, batch)
  int swap_staged;                // launcher: the swapped GLU tile leaves through shared memory and TMA stores (map tm_out0)
  int rm_seg, rm_slot;            // launcher: segment whose full tiles leave through shared memory and a TMA store (row-major
                                  // bf16; BN = 128 plain kernel), and the output map it uses; rm_seg < 0: none
  int xpose;                      // launcher (BN = 128 plain kernel, one row-major float32 segment with gate / residual):
                                  // every warp moves its 32 x 32 chunk of gate, residual and output through a private
                                  // shared-memory tile, so that global memory sees whole 128-byte rows
  int glu;                        // GluMode; with GLU a BN tile holds BN/2 values then BN/2 gates
  int swap;                       // launcher: channel-major GLU output computed in the swapped orientation (see SWAP)
  int a_mn_major;                 // launcher: the A operand is stored K-outer ([k][row], rows contiguous) and read MN-major
  int k_inner;                    // launcher: != 0: both operands store K in pieces of k_inner elements (a multiple of the K
                                  // tile) that lie `s_k_hi` apart: K index = (k / k_inner, k % k_inner), five-dimensional maps
  const float2* row_stats;        // optional LayerNorm fold: out = rstd[row] * (acc - mean[row] * col_s1[col]) + col_s0[col]
  const float* col_s1;            //   (mean, rstd) per flat row; col_s1 = sum_k W'[col][k], col_s0 = sum_k beta[k] W[col][k]
  const float* col_s0;            //   with W' = gamma * W the matrix actually multiplied (applied before gate / residual)
  int swap_col_begin;             // launcher (BN = 128, plain epilogue): tiles whose first column is >= this hold channel-major
                                  // segments only and are computed in the swapped orientation too (INT_MAX: none)
  int nseg;
  EpiSeg seg[3];
  const unsigned char* rowmask;   // optional 0/1 mask multiplied into segment rows flagged below
  long long m_n, m_o, m_b;
  int mask_segs;                  // bit i: apply rowmask to segment i
  const float* col_bias;          // optional, per output column, added before everything else
  int precise;                    // fp32-accurate mode: exact sigmoid, fp32 gate logits, split stores
  int k_main_blocks;              // precise: the first k_main_blocks k-blocks (the x0*w0 products) accumulate in their own
                                  // TMEM accumulator, the five correction blocks in a second one; the epilogue adds the
                                  // two in fp32.  The tensor core truncates on every accumulation step, relative to the
                                  // accumulator's magnitude: keeping the small corrections apart keeps their error small
  const __nv_bfloat16* gate;      // optional: seg 0 value *= sigmoid(gate[...]), addressed with seg 0 strides
                                  // (points at float logits when `precise`)
  long long g_col, g_n, g_o, g_b;
  int stages;                     // depth of the operand ring (launcher)
  int aux;                        // 1: gate / residual tiles are prefetched into shared memory by TMA (launcher)
  int aux_gate, aux_resid;        // which of the two the prefetch covers
  long long* trace;               // debugging aid: CTA 0 stores clock64() stamps per tile here when non-null
  const void* resid;              // optional: seg 0 value += resid[...] (same dtype and strides as seg 0 dst)
  const float* resid_scale;       // optional, per output column: seg 0 value += resid_scale[col] * resid[...] instead
                                  // (the state decay of the trunk's recurrence, z <- a * z + Linear(...))
};

static constexpr int kBM = 128;
static constexpr int kBK = 64;   // bf16 elements = 128 bytes = one swizzle span
static constexpr int kEpiWarps = 8;  // two warps per TMEM lane quadrant, each taking every other 32-column chunk
static constexpr int kGemmThreads = 64 + 32 * kEpiWarps;

template <int BN>
struct GemmCfg {
  static constexpr int kAStage = kBM * kBK * 2;
  static constexpr int kBStage = BN * kBK * 2;
  static constexpr int kStageBytes = kAStage + kBStage;
  static constexpr int kMaxStages = 8;
  // per group of 4 epilogue warps: 2 slabs of [32 channels][128 rows] bf16 -- or, in the BN = 128 kernel, two whole row-major
  // output tiles (two 64-column boxes of [128 rows][128 bytes] each) on their way to a TMA store
  static constexpr int kSlabBytes = (kEpiWarps / 4) * 2 * 32 * kBM * 2;
  static constexpr int kRowTileBytes = kBM * 128 * 2;
  static constexpr int kStagingBytes = (BN == 128) ? 2 * kRowTileBytes : kSlabBytes;
  // the GLU kernel at BN = 256 writes 128 output columns per tile: the same two row-major tile buffers
  static constexpr int kGluStagingBytes = (BN == 256) ? 2 * kRowTileBytes : kStagingBytes;
  // swapped-orientation GLU kernel (BN = 256): the tile's position mask (1 KB, two accumulators) and two whole
  // channel-major output tiles ([2 boxes of 64 positions][128 channels][128 bytes])
  static constexpr int kSwapStagingBytes = 1024 + 2 * kRowTileBytes;
  static constexpr int kBarrierBytes = 512;
  static constexpr int kSmemBytes = 232448 - 1024;        // everything an SM offers one CTA
  // after the operand ring comes EITHER the channel-major staging slabs OR two buffers of prefetched
  // gate + residual tiles (128 rows x BN columns bf16 each); the launcher picks the ring depth accordingly
  static constexpr int kAuxTileBytes = kBM * BN * 2;
  static constexpr int kAuxBytes = 2 * 2 * kAuxTileBytes;
  static constexpr int stages_for(int extra_bytes) {
    const int fit = (kSmemBytes - 1024 - extra_bytes - kBarrierBytes) / kStageBytes;
    return fit < kMaxStages ? fit : kMaxStages;
  }
  static constexpr int kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;
};

// The GLU epilogues of the bf16 kernels get their gate operands halved by the weight packing (exact in bf16):
//   v sigmoid(g)   = v' + v' tanh(g')      with v' = v / 2, g' = g / 2
//   a sigmoid(a) g = (a' + a' tanh(a')) g  with a' = a / 2
// one MUFU op and one fused multiply-add per gate.
__device__ __forceinline__ float tanh_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
  return t;
}
__device__ __forceinline__ float glu_half(float v_half, float g_half) { return fmaf(v_half, tanh_fast(g_half), v_half); }

// sigmoid(x) = 0.5 tanh(x / 2) + 0.5: one MUFU op instead of an exp2 and a reciprocal
__device__ __forceinline__ float sigmoidf_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(t, 0.5f, 0.5f);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float sigmoidf_exact(float x) { return 1.0f / (1.0f + __expf(-x)); }

// x = x0 + x1 + x2 with three bf16 parts (24 mantissa bits): the operands of the fp32-accurate GEMMs.
__device__ __forceinline__ void split3(float x, __nv_bfloat16& x0, __nv_bfloat16& x1, __nv_bfloat16& x2) {
  x0 = __float2bfloat16_rn(x);
  const float r1 = x - __bfloat162float(x0);
  x1 = __float2bfloat16_rn(r1);
  x2 = __float2bfloat16_rn(r1 - __bfloat162float(x1));
}

// Split store of 32 values of one row: six copies, s_part elements apart (see EpiSeg::split).
__device__ __forceinline__ void epi_store_split(const EpiSeg& sg, long long row_off, int col_local, const float (&v)[32],
                                                bool row_ok) {
  if (!row_ok) return;
  const int nvalid = min(32, sg.ncols - col_local);
  __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(sg.dst) + row_off + static_cast<long long>(col_local) * sg.s_col;
#pragma unroll 4
  for (int i = 0; i < 32; ++i) {
    if (i >= nvalid) break;
    __nv_bfloat16 x0, x1, x2;
    split3(v[i], x0, x1, x2);
    __nv_bfloat16* e = d + static_cast<long long>(i) * sg.s_col;
    if (sg.split == 1) {
      e[0] = x0; e[sg.s_part] = x0; e[2 * sg.s_part] = x1; e[3 * sg.s_part] = x1; e[4 * sg.s_part] = x0; e[5 * sg.s_part] = x2;
    } else {
      e[0] = x0; e[sg.s_part] = x1; e[2 * sg.s_part] = x0; e[3 * sg.s_part] = x1; e[4 * sg.s_part] = x2; e[5 * sg.s_part] = x0;
    }
  }
}

// 32-byte global store (one full sector per thread and instruction)
__device__ __forceinline__ void st_global_v8(void* ptr, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t a4,
                                             uint32_t a5, uint32_t a6, uint32_t a7) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(a0), "r"(a1), "r"(a2), "r"(a3),
               "r"(a4), "r"(a5), "r"(a6), "r"(a7)
               : "memory");
}

// Store 32 consecutive output values of one row.
__device__ __forceinline__ void epi_store_chunk(const EpiSeg& sg, long long row_off, int col_local, const float (&v)[32],
                                                bool row_ok) {
  if (!row_ok) return;
  const int nvalid = min(32, sg.ncols - col_local);
  if (nvalid <= 0) return;
  if (sg.vec && nvalid == 32) {
    if (sg.out_fp32) {
      float* d = reinterpret_cast<float*>(sg.dst) + row_off + col_local;
      if ((reinterpret_cast<uintptr_t>(d) & 31) == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          st_global_v8(d + 8 * i, __float_as_uint(v[8 * i]), __float_as_uint(v[8 * i + 1]), __float_as_uint(v[8 * i + 2]),
                       __float_as_uint(v[8 * i + 3]), __float_as_uint(v[8 * i + 4]), __float_as_uint(v[8 * i + 5]),
                       __float_as_uint(v[8 * i + 6]), __float_as_uint(v[8 * i + 7]));
      } else {
        float4* d4 = reinterpret_cast<float4*>(d);
#pragma unroll
        for (int i = 0; i < 8; ++i) d4[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      }
    } else {
      __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(sg.dst) + row_off + col_local;
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) w[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
      if ((reinterpret_cast<uintptr_t>(d) & 31) == 0) {
        st_global_v8(d, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
        st_global_v8(d + 16, w[8], w[9], w[10], w[11], w[12], w[13], w[14], w[15]);
      } else {
        uint4* d4 = reinterpret_cast<uint4*>(d);
#pragma unroll
        for (int i = 0; i < 4; ++i) d4[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
      }
    }
    return;
  }
  // scalar path: per column; coalesced across the warp's lanes when s_n == 1 (channel-major output)
  if (sg.out_fp32) {
    float* d = reinterpret_cast<float*>(sg.dst) + row_off + static_cast<long long>(col_local) * sg.s_col;
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < nvalid) d[static_cast<long long>(i) * sg.s_col] = v[i];
  } else {
    __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(sg.dst) + row_off + static_cast<long long>(col_local) * sg.s_col;
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < nvalid) d[static_cast<long long>(i) * sg.s_col] = __float2bfloat16_rn(v[i]);
  }
}

// A tile index as (n tile, row block, outer, batch).  The persistent loops step by the grid size; stepping the mixed-radix
// digits with carries replaces five integer divisions per tile and role (which cost the epilogue warps about 800 cycles
// of every 4500-cycle tile).
struct TileIdx {
  int n_tile, nb, o, b;
};
__device__ __forceinline__ TileIdx tile_decompose(int tile, const GemmParams& p) {
  TileIdx t;
  const int m_tile = tile / p.num_n_tiles;
  t.n_tile = tile - m_tile * p.num_n_tiles;
  t.nb = m_tile % p.n_blocks;
  const int rest = m_tile / p.n_blocks;
  t.o = rest % p.o_extent;
  t.b = rest / p.o_extent;
  return t;
}
// t += grid size, whose digits the launcher put into the parameters (each below its radix)
__device__ __forceinline__ void tile_advance(TileIdx& t, const GemmParams& p) {
  t.n_tile += p.step_n_tile;
  int carry = t.n_tile >= p.num_n_tiles ? 1 : 0;
  t.n_tile -= carry ? p.num_n_tiles : 0;
  t.nb += p.step_nb + carry;
  carry = t.nb >= p.n_blocks ? 1 : 0;
  t.nb -= carry ? p.n_blocks : 0;
  t.o += p.step_o + carry;
  carry = t.o >= p.o_extent ? 1 : 0;
  t.o -= carry ? p.o_extent : 0;
  t.b += p.step_b + carry;
}

// GLU and AUX are compile-time so that each variant carries only its own epilogue code (and registers):
//   GLU  the tile holds values and gates (p.glu says which activation);
//   AUX  gate logits / residual come from shared-memory tiles prefetched by the producer.
//   PRECISE  fp32-accurate mode (operands are bf16 triple splits concatenated along K, see split3): exact
//            sigmoid, fp32 gate logits, split stores.
//   SWAP  channel-major GLU output (the triangle-multiplication operands): the tensor core computes the TRANSPOSED tile,
//         D[channel][position] = W[channel][:] . X[position][:], i.e. the 128 value rows and the 128 gate rows of the weight
//         tile are the M operands of two N=128 MMAs and the 128 positions are the N operand.  A thread then holds
//         consecutive positions of ONE channel and writes them with 32-byte stores: no transpose through shared memory.
template <int BN, bool GLU, bool AUX, bool PRECISE, bool SWAP = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_out0, const __grid_constant__ CUtensorMap tm_out1,
                 const GemmParams p) {
  // tm_out0 / tm_out1: TMA-store maps of channel-major segments, or (p.aux) the gate / residual load maps
  using Cfg = GemmCfg<BN>;
  const int kStages = p.stages;
  constexpr int OUT_BN_GLU = BN / 2;
  constexpr int ACC_COLS = PRECISE ? 2 * BN : BN;  // precise: main accumulator, then the correction accumulator
  static_assert(!PRECISE || BN <= 128, "the fp32-accurate variant needs four accumulators of BN columns");
  static_assert(!SWAP || (BN == 256 && GLU && !AUX && !PRECISE), "the swapped orientation exists for the BN = 256 GLU tile");
  constexpr bool kPlain128 = (BN == 128 && !GLU && !AUX && !PRECISE);  // the variant that may swap single tiles

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_a = smem;
  uint8_t* s_b = smem + kStages * Cfg::kAStage;
  uint8_t* s_stage_out = smem + kStages * Cfg::kStageBytes;  // [group of 4 epilogue warps][2][32 channels][128 rows] bf16 ...
  uint8_t* s_aux = s_stage_out;                               // ... or [2 buffers][gate, resid][2 halves? BN/64][128 x 64] bf16
  uint64_t* bars = reinterpret_cast<uint64_t*>(
      s_stage_out + (AUX ? Cfg::kAuxBytes : (SWAP ? Cfg::kSwapStagingBytes : (GLU ? Cfg::kGluStagingBytes : Cfg::kStagingBytes))));
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + Cfg::kMaxStages;
  uint64_t* tmem_full = bars + 2 * Cfg::kMaxStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* aux_full = tmem_empty + 2;   // [2]
  uint64_t* aux_empty = aux_full + 2;    // [2], one arrival per epilogue warp
  uint64_t* cm_bar = aux_empty + 2;      // [2 groups][slab free, slab written], 128 arrivals each
  uint64_t* rm_bar = cm_bar + 4;         // [2 staging buffers]: row-major tile written, one arrival per epilogue thread
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(rm_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_k = (p.k_extent + kBK - 1) / kBK;
  const int total_tiles = p.num_m_tiles * p.num_n_tiles;
  long long* trace = (p.trace != nullptr && blockIdx.x == 0) ? p.trace : nullptr;
#ifdef KFB_DEBUG_TRACE
#define KFB_GSTAMP(slot) do { if (trace != nullptr && (slot) < 512) trace[slot] = clock64(); } while (0)
#else
#define KFB_GSTAMP(slot) do { (void)trace; } while (0)
#endif

  if (threadIdx.x == 0) {
    KFB_GSTAMP(0);
    ptx::prefetch_tmap(&tm_a);
    ptx::prefetch_tmap(&tm_b);
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&tmem_full[a], 1);
      ptx::mbar_init(&tmem_empty[a], 32 * kEpiWarps);
      ptx::mbar_init(&aux_full[a], 1);
      ptx::mbar_init(&aux_empty[a], kEpiWarps);
    }
    for (int a = 0; a < 4; ++a) ptx::mbar_init(&cm_bar[a], 128);
    for (int a = 0; a < 2; ++a) ptx::mbar_init(&rm_bar[a], 32 * kEpiWarps);
    ptx::fence_barrier_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, PRECISE ? 2 * Cfg::kTmemCols : Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;  // ring position, advanced without divisions (the ring depth is a run-time value)
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int m_tile = tile / p.num_n_tiles;
        const int n_tile = tile - m_tile * p.num_n_tiles;
        const int nb = m_tile % p.n_blocks;
        const int rest = m_tile / p.n_blocks;
        const int o = rest % p.o_extent;
        const int b = rest / p.o_extent;
        const int bb = p.b_batched ? b : 0;
        const int b_col_hi = (n_tile * BN) / p.b_col_inner;
        const int b_col_lo = n_tile * BN - b_col_hi * p.b_col_inner;
        if (AUX) {
          // gate / residual tiles of this output tile, one tile ahead of the epilogue
          const uint32_t ti = (tile - blockIdx.x) / gridDim.x;
          const int ab = ti & 1;
          if (!ptx::mbar_wait(&aux_empty[ab], ((ti >> 1) & 1) ^ 1, 106)) { ok = false; break; }
          uint8_t* dst = s_aux + ab * (2 * Cfg::kAuxTileBytes);
          ptx::mbar_expect_tx(&aux_full[ab], (p.aux_gate + p.aux_resid) * Cfg::kAuxTileBytes);
#pragma unroll
          for (int hcol = 0; hcol < BN / 64; ++hcol) {
            if (p.aux_gate)
              ptx::tma_load_4d(dst + hcol * (kBM * 128), &tm_out0, &aux_full[ab], n_tile * BN + hcol * 64, nb * kBM, o, b);
            if (p.aux_resid)
              ptx::tma_load_4d(dst + Cfg::kAuxTileBytes + hcol * (kBM * 128), &tm_out1, &aux_full[ab], n_tile * BN + hcol * 64,
                               nb * kBM, o, b);
          }
        }
        for (int kb = 0; kb < num_k; ++kb) {
          if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1, 101)) { ok = false; break; }
          ptx::mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          if (p.a_mn_major) {
            // two boxes of [64 k][64 rows]: 128-byte rows of consecutive rows (positions), one per k index
            ptx::tma_load_4d(s_a + stage * Cfg::kAStage, &tm_a, &full_bar[stage], nb * kBM, kb * kBK, o, b);
            ptx::tma_load_4d(s_a + stage * Cfg::kAStage + Cfg::kAStage / 2, &tm_a, &full_bar[stage], nb * kBM + 64, kb * kBK, o, b);
          } else if (p.k_inner) {
            const int k_hi = (kb * kBK) / p.k_inner;
            const int k_lo = kb * kBK - k_hi * p.k_inner;
            ptx::tma_load_5d(s_a + stage * Cfg::kAStage, &tm_a, &full_bar[stage], k_lo, nb * kBM, o, k_hi, b);
            ptx::tma_load_5d(s_b + stage * Cfg::kBStage, &tm_b, &full_bar[stage], k_lo, b_col_lo, b_col_hi, k_hi, bb);
            if (++stage == kStages) { stage = 0; phase ^= 1; }
            continue;
          } else
          ptx::tma_load_4d(s_a + stage * Cfg::kAStage, &tm_a, &full_bar[stage], kb * kBK, nb * kBM, o, b);
          ptx::tma_load_4d(s_b + stage * Cfg::kBStage, &tm_b, &full_bar[stage], kb * kBK, b_col_lo, b_col_hi, bb);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        KFB_GSTAMP(4 + (tile / gridDim.x) * 4 + 3);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_idesc(kBM, BN, /*bf16*/ 1);
      uint32_t tile_iter = 0;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++tile_iter) {
        const uint32_t acc = tile_iter & 1;
        const uint32_t acc_phase = (tile_iter >> 1) & 1;
        const int n_tile_mma = tile % p.num_n_tiles;
        if (!ptx::mbar_wait(&tmem_empty[acc], acc_phase ^ 1, 102)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!ptx::mbar_wait(&full_bar[stage], phase, 103)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          // one descriptor per stage; inside the 128-byte swizzle span only the address field advances
          const uint64_t a_desc = ptx::make_kmajor_desc<128>(ptx::smem_u32(s_a + stage * Cfg::kAStage));
          const uint64_t b_desc = ptx::make_kmajor_desc<128>(ptx::smem_u32(s_b + stage * Cfg::kBStage));
          const bool corr = PRECISE && kb >= p.k_main_blocks;
          const uint32_t d_acc = corr ? d_tmem + BN : d_tmem;
          const bool first = corr ? (kb == p.k_main_blocks) : (kb == 0);
          if constexpr (SWAP) {
            // value rows (first 128 rows of the weight stage) -> columns 0..127, gate rows -> columns 128..255
            constexpr uint32_t idesc_sw = ptx::make_idesc(kBM, 128, /*bf16*/ 1);
            const uint64_t g_desc = b_desc + ((128 * 128) >> 4);
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k) {
              ptx::mma_f16_ss(d_acc, b_desc + k * 2, a_desc + k * 2, idesc_sw, (first && k == 0) ? 0u : 1u);
              ptx::mma_f16_ss(d_acc + 128, g_desc + k * 2, a_desc + k * 2, idesc_sw, (first && k == 0) ? 0u : 1u);
            }
          } else if (p.a_mn_major) {
            // A as [k][rows]: MN-major, 128-byte swizzled rows; 8 k-rows are 1024 bytes apart, the next 64 rows
            // (positions) half a stage further; a K=16 step advances by 16 k-rows = 2048 bytes
            const uint64_t am_desc = static_cast<uint64_t>((ptx::smem_u32(s_a + stage * Cfg::kAStage) & 0x3ffff) >> 4) |
                                     (static_cast<uint64_t>((Cfg::kAStage / 2) >> 4) << 16) |
                                     (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              ptx::mma_f16_ss(d_acc, am_desc + k * (2048 >> 4), b_desc + k * 2, idesc | (1u << 15), (first && k == 0) ? 0u : 1u);
          } else {
            // (plain BN = 128 tiles of channel-major segments: operands exchanged, D[channel][position])
            const bool sw = kPlain128 && n_tile_mma * BN >= p.swap_col_begin;
            const uint64_t m_desc = sw ? b_desc : a_desc, n_desc = sw ? a_desc : b_desc;
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              ptx::mma_f16_ss(d_acc, m_desc + k * 2, n_desc + k * 2, idesc, (first && k == 0) ? 0u : 1u);
          }
          ptx::tc_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) ptx::tc_commit(&tmem_full[acc]);
        KFB_GSTAMP(4 + tile_iter * 4 + 2);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const int chunk_phase = (warp - 2) >> 2;  // which of the interleaved column chunks this warp takes
    uint32_t staging_use = 0;
    uint32_t rm_use = 0;  // row-major tiles sent through the staging buffers so far (the same count in every epilogue thread)
    const int r = quad * 32 + lane;
    uint32_t tile_iter = 0;
    bool ok = true;
    // the row-mask byte of a tile is fetched one tile ahead, so that its latency never shows in the epilogue: the load is
    // issued here as it stands (volatile asm: the compiler may not sink it to its use) and only its raw byte is kept; the
    // comparison that consumes it happens one tile later
    auto load_mask = [&](int tile, const TileIdx& t) -> uint32_t {
      if (p.rowmask == nullptr || tile >= total_tiles) return 1u;
      const int n = t.nb * kBM + r;
      if (n >= p.n_extent) return 1u;
      uint32_t raw;
      asm volatile("ld.global.nc.u8 %0, [%1];" : "=r"(raw)
                   : "l"(p.rowmask + static_cast<long long>(t.b) * p.m_b + static_cast<long long>(t.o) * p.m_o +
                         static_cast<long long>(n) * p.m_n));
      return raw;
    };
    TileIdx tile_cur = tile_decompose(static_cast<int>(blockIdx.x), p);
    uint32_t mask_next = load_mask(blockIdx.x, tile_cur);
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++tile_iter, tile_advance(tile_cur, p)) {
      const int n_tile = tile_cur.n_tile, nb = tile_cur.nb, o = tile_cur.o, b = tile_cur.b;
      const int n = nb * kBM + r;
      const bool row_ok = n < p.n_extent;
      const float mask_v = mask_next ? 1.0f : 0.0f;
      if (p.rowmask != nullptr) {   // the next tile's index only lives until its mask load is issued
        TileIdx peek = tile_cur;
        tile_advance(peek, p);
        mask_next = load_mask(tile + gridDim.x, peek);
      }
      const uint32_t acc = tile_iter & 1;
      const uint32_t acc_phase = (tile_iter >> 1) & 1;
      if (!ptx::mbar_wait(&tmem_full[acc], acc_phase, 104)) { ok = false; break; }
      if (threadIdx.x == 64) KFB_GSTAMP(4 + tile_iter * 4 + 0);
      ptx::tc_fence_after_sync();
      const uint8_t* aux_tile = s_aux + (tile_iter & 1) * (2 * Cfg::kAuxTileBytes);
      if (AUX && !ptx::mbar_wait(&aux_full[tile_iter & 1], (tile_iter >> 1) & 1, 107)) { ok = false; break; }
      const uint32_t t_row = tmem_base + acc * ACC_COLS + (static_cast<uint32_t>(quad * 32) << 16);

      constexpr int out_bn = GLU ? OUT_BN_GLU : BN;
      const int out_col_tile = n_tile * out_bn;
      if constexpr (SWAP) {
        // lanes are channels, columns are the tile's 128 positions.  The position mask of the tile goes through shared
        // memory: thread r of the first four epilogue warps holds the mask of position r (fetched a tile ahead).
        float* s_maskf = reinterpret_cast<float*>(s_stage_out) + acc * kBM;
        if (chunk_phase == 0) {
          s_maskf[r] = mask_v;
          ptx::mbar_arrive(&cm_bar[acc]);
        }
        if (!ptx::mbar_wait(&cm_bar[acc], acc_phase, 108)) { ok = false; break; }
        const EpiSeg& sg = p.seg[0];
        const int ch = out_col_tile + r;  // output channel of this lane
        __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(sg.dst) + static_cast<long long>(ch) * sg.s_col +
                              static_cast<long long>(b) * sg.s_b + static_cast<long long>(o) * sg.s_o;
        bool swap_done = false;
        if (p.swap_staged) {
          // staged tile: the lane's 64 positions go by as four pieces of 16, the tensor-memory load of the next piece issued
          // before the arithmetic of the current one (one exposed round trip per tile instead of two)
          constexpr int kPieces = 2 * (kBM / (32 * (kEpiWarps / 4)));
          uint8_t* buf = s_stage_out + 1024 + (rm_use & 1) * Cfg::kRowTileBytes;
          auto piece_col = [&](int i) { return chunk_phase * 32 + (i >> 1) * (32 * (kEpiWarps / 4)) + (i & 1) * 16; };
          uint32_t va[16], ga[16], vb[16], gb[16];
          ptx::tmem_ld_32x32b_x16(t_row + piece_col(0), va);
          ptx::tmem_ld_32x32b_x16(t_row + 128 + piece_col(0), ga);
          auto finish_piece = [&](int c, const uint32_t (&vv)[16], const uint32_t (&gg)[16]) {
            uint32_t w[8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 m4 = *reinterpret_cast<const float4*>(s_maskf + c + 4 * q);
              const float mk4[4] = {m4.x, m4.y, m4.z, m4.w};
#pragma unroll
              for (int i = 0; i < 4; i += 2)
                w[q * 2 + (i >> 1)] =
                    pack_bf16x2(glu_half(__uint_as_float(vv[4 * q + i]), __uint_as_float(gg[4 * q + i])) * mk4[i],
                                glu_half(__uint_as_float(vv[4 * q + i + 1]), __uint_as_float(gg[4 * q + i + 1])) * mk4[i + 1]);
            }
            uint8_t* rowp = buf + (c >> 6) * (Cfg::kRowTileBytes / 2) + r * 128;
            const int piece = (c & 63) >> 3;
            *reinterpret_cast<uint4*>(rowp + (((piece) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4*>(rowp + (((piece + 1) ^ (r & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
          };
#pragma unroll
          for (int i = 0; i < kPieces; i += 2) {
            ptx::tmem_ld_wait();
            if (i + 1 < kPieces) {
              ptx::tmem_ld_32x32b_x16(t_row + piece_col(i + 1), vb);
              ptx::tmem_ld_32x32b_x16(t_row + 128 + piece_col(i + 1), gb);
            }
            finish_piece(piece_col(i), va, ga);
            ptx::tmem_ld_wait();
            if (i + 2 < kPieces) {
              ptx::tmem_ld_32x32b_x16(t_row + piece_col(i + 2), va);
              ptx::tmem_ld_32x32b_x16(t_row + 128 + piece_col(i + 2), ga);
            }
            if (i + 1 < kPieces) finish_piece(piece_col(i + 1), vb, gb);
          }
          swap_done = true;
        }
        if (!swap_done)
#pragma unroll 1
        for (int c = chunk_phase * 32; c < kBM; c += 32 * (kEpiWarps / 4)) {
          uint32_t raw[32], rawg[32];
          ptx::tmem_ld_32x32b_x32(t_row + c, raw);
          ptx::tmem_ld_32x32b_x32(t_row + 128 + c, rawg);
          float mk[32];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 m4 = *reinterpret_cast<const float4*>(s_maskf + c + 4 * q);
            mk[4 * q] = m4.x; mk[4 * q + 1] = m4.y; mk[4 * q + 2] = m4.z; mk[4 * q + 3] = m4.w;
          }
          ptx::tmem_ld_wait();
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float v0 = glu_half(__uint_as_float(raw[i]), __uint_as_float(rawg[i])) * mk[i];
            const float v1 = glu_half(__uint_as_float(raw[i + 1]), __uint_as_float(rawg[i + 1])) * mk[i + 1];
            w[i >> 1] = pack_bf16x2(v0, v1);
          }
          const int n0 = nb * kBM + c;
          if (p.swap_staged) {
            // this channel's 32 positions into the staged tile: box c / 64, row = channel, 128-byte rows with the copy
            // engine's 16-byte swizzle (conflict-free 16-byte stores)
            uint8_t* rowp = s_stage_out + 1024 + (rm_use & 1) * Cfg::kRowTileBytes + (c >> 6) * (Cfg::kRowTileBytes / 2) + r * 128;
            const int piece = (c & 63) >> 3;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
              *reinterpret_cast<uint4*>(rowp + (((piece + q4) ^ (r & 7)) << 4)) =
                  make_uint4(w[4 * q4], w[4 * q4 + 1], w[4 * q4 + 2], w[4 * q4 + 3]);
            continue;
          }
          if (ch < sg.ncols) {
            __nv_bfloat16* d = drow + n0;
            if (n0 + 32 <= p.n_extent && (reinterpret_cast<uintptr_t>(d) & 31) == 0) {
              st_global_v8(d, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
              st_global_v8(d + 16, w[8], w[9], w[10], w[11], w[12], w[13], w[14], w[15]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (n0 + i < p.n_extent)
                  d[i] = __ushort_as_bfloat16(static_cast<unsigned short>((i & 1) ? (w[i >> 1] >> 16) : (w[i >> 1] & 0xffffu)));
            }
          }
        }
        if (p.swap_staged) {
          // whole rows of the channel-major tile leave through the copy engine (a thread's own 32-byte stores cost one
          // memory request per sector); two buffers alternate as in the row-major path below
          ptx::fence_proxy_async_smem();
          const bool issuer = (quad == 0 && chunk_phase == 0 && lane == 0);
          if (issuer) ptx::tma_store_wait_read();
          ptx::mbar_arrive(&rm_bar[rm_use & 1]);
          if (!ptx::mbar_wait(&rm_bar[rm_use & 1], (rm_use >> 1) & 1, 111)) { ok = false; break; }
          if (issuer) {
            const uint8_t* buf = s_stage_out + 1024 + (rm_use & 1) * Cfg::kRowTileBytes;
            ptx::tma_store_4d(&tm_out0, buf, nb * kBM, o, out_col_tile, b);
            if (nb * kBM + 64 < p.n_extent)
              ptx::tma_store_4d(&tm_out0, buf + Cfg::kRowTileBytes / 2, nb * kBM + 64, o, out_col_tile, b);
            ptx::tma_store_commit();
          }
          ++rm_use;
        }
      } else if (kPlain128 && out_col_tile >= p.swap_col_begin) {
        // a tile of channel-major segments, computed swapped: this lane is output column (channel) out_col_tile + r, the
        // tile's columns are its 128 positions.  The launcher guarantees that the tile lies inside one segment.
        int si = 0;
        if (p.nseg > 1 && out_col_tile >= p.seg[1].col_begin) si = 1;
        if (p.nseg > 2 && out_col_tile >= p.seg[2].col_begin) si = 2;
        const EpiSeg& sg = p.seg[si];
        const int ch_local = out_col_tile + r - sg.col_begin;
        const bool lane_ok = ch_local < sg.ncols;
        const float bias_v = (p.col_bias != nullptr && lane_ok) ? p.col_bias[out_col_tile + r] : 0.0f;
        __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(sg.dst) + static_cast<long long>(lane_ok ? ch_local : 0) * sg.s_col +
                              static_cast<long long>(b) * sg.s_b + static_cast<long long>(o) * sg.s_o;
#pragma unroll 1
        for (int c = chunk_phase * 32; c < kBM; c += 32 * (kEpiWarps / 4)) {
          uint32_t raw[32];
          ptx::tmem_ld_32x32b_x32(t_row + c, raw);
          ptx::tmem_ld_wait();
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            w[i >> 1] = pack_bf16x2(__uint_as_float(raw[i]) + bias_v, __uint_as_float(raw[i + 1]) + bias_v);
          const int n0 = nb * kBM + c;
          if (lane_ok) {
            __nv_bfloat16* d = drow + n0;
            if (n0 + 32 <= p.n_extent && (reinterpret_cast<uintptr_t>(d) & 31) == 0) {
              st_global_v8(d, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
              st_global_v8(d + 16, w[8], w[9], w[10], w[11], w[12], w[13], w[14], w[15]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (n0 + i < p.n_extent)
                  d[i] = __ushort_as_bfloat16(static_cast<unsigned short>((i & 1) ? (w[i >> 1] >> 16) : (w[i >> 1] & 0xffffu)));
            }
          }
        }
      } else {
      // Fast path of the plain kernel: a tile that lies inside one row-major bf16 segment and needs nothing but the
      // conversion and a column bias (the q / k / g columns of the attention projections, plain projections): none of the
      // per-chunk bookkeeping of the general loop below.
      bool tile_done = false;
      if constexpr (!GLU && !AUX && !PRECISE && BN >= 128) {
        int si = 0;
        if (p.nseg > 1 && out_col_tile >= p.seg[1].col_begin) si = 1;
        if (p.nseg > 2 && out_col_tile >= p.seg[2].col_begin) si = 2;
        const EpiSeg& sg = p.seg[si];
        const bool plain = sg.vec && !sg.out_fp32 && sg.tma_slot < 0 && out_col_tile + BN <= sg.col_begin + sg.ncols &&
                           (reinterpret_cast<uintptr_t>(p.col_bias) & 15) == 0 && p.row_stats == nullptr &&
                           !((p.mask_segs >> si) & 1) &&
                           (si != 0 || (p.gate == nullptr && p.resid == nullptr));
        if (plain) {
          __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(sg.dst) + static_cast<long long>(b) * sg.s_b +
                                static_cast<long long>(o) * sg.s_o + static_cast<long long>(n) * sg.s_n +
                                (out_col_tile - sg.col_begin);
#pragma unroll 1
          for (int c = chunk_phase * 32; c < BN; c += 128) {
            uint32_t r0[32], r1[32];
            ptx::tmem_ld_32x32b_x32(t_row + c, r0);
            ptx::tmem_ld_32x32b_x32(t_row + c + 64, r1);
            ptx::tmem_ld_wait();
            if (p.col_bias != nullptr) {   // per output column, the same for every row: uniform 16-byte loads
              const float4* b0 = reinterpret_cast<const float4*>(p.col_bias + out_col_tile + c);
              const float4* b1 = reinterpret_cast<const float4*>(p.col_bias + out_col_tile + c + 64);
#pragma unroll
              for (int q4 = 0; q4 < 8; ++q4) {
                const float4 u0 = __ldg(b0 + q4), u1 = __ldg(b1 + q4);
                r0[4 * q4] = __float_as_uint(__uint_as_float(r0[4 * q4]) + u0.x);
                r0[4 * q4 + 1] = __float_as_uint(__uint_as_float(r0[4 * q4 + 1]) + u0.y);
                r0[4 * q4 + 2] = __float_as_uint(__uint_as_float(r0[4 * q4 + 2]) + u0.z);
                r0[4 * q4 + 3] = __float_as_uint(__uint_as_float(r0[4 * q4 + 3]) + u0.w);
                r1[4 * q4] = __float_as_uint(__uint_as_float(r1[4 * q4]) + u1.x);
                r1[4 * q4 + 1] = __float_as_uint(__uint_as_float(r1[4 * q4 + 1]) + u1.y);
                r1[4 * q4 + 2] = __float_as_uint(__uint_as_float(r1[4 * q4 + 2]) + u1.z);
                r1[4 * q4 + 3] = __float_as_uint(__uint_as_float(r1[4 * q4 + 3]) + u1.w);
              }
            }
            uint32_t w0[16], w1[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              w0[i] = pack_bf16x2(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]));
              w1[i] = pack_bf16x2(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1]));
            }
            if constexpr (BN == 128) {
              if (si == p.rm_seg) {
                // Through shared memory: a thread's 32-byte stores to 32 different rows cost one memory request per
                // sector; the copy engine writes whole rows of the tile instead.  Two buffers alternate; a buffer is
                // reused two staged tiles later, after the issuing thread has seen its store read it (checked before
                // the barrier of the tile in between).
                uint8_t* buf = s_stage_out + (rm_use & 1) * Cfg::kRowTileBytes;
                uint8_t* row0 = buf + r * 128;                              // columns 0..63 of this row
                uint8_t* row1 = buf + Cfg::kRowTileBytes / 2 + r * 128;     // columns 64..127
                const int piece = (c >> 3);                                 // first 16-byte piece: 0 or 4
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                  const int phys = ((piece + q4) ^ (r & 7)) << 4;
                  *reinterpret_cast<uint4*>(row0 + phys) = make_uint4(w0[4 * q4], w0[4 * q4 + 1], w0[4 * q4 + 2], w0[4 * q4 + 3]);
                  *reinterpret_cast<uint4*>(row1 + phys) = make_uint4(w1[4 * q4], w1[4 * q4 + 1], w1[4 * q4 + 2], w1[4 * q4 + 3]);
                }
                ptx::fence_proxy_async_smem();
                const bool issuer = (quad == 0 && chunk_phase == 0 && lane == 0);
                if (issuer) ptx::tma_store_wait_read();   // the previous staged tile's store has read the other buffer
                ptx::mbar_arrive(&rm_bar[rm_use & 1]);
                if (!ptx::mbar_wait(&rm_bar[rm_use & 1], (rm_use >> 1) & 1, 110)) { ok = false; break; }
                if (issuer) {
                  const CUtensorMap* tm = p.rm_slot == 0 ? &tm_out0 : &tm_out1;
                  const int col0 = out_col_tile - sg.col_begin;
                  ptx::tma_store_4d(tm, buf, col0, nb * kBM, o, b);
                  if (col0 + 64 < sg.ncols) ptx::tma_store_4d(tm, buf + Cfg::kRowTileBytes / 2, col0 + 64, nb * kBM, o, b);
                  ptx::tma_store_commit();
                }
                ++rm_use;
                continue;
              }
            }
            if (row_ok) {
              __nv_bfloat16* d = drow + c;
              if ((reinterpret_cast<uintptr_t>(d) & 31) == 0) {
                st_global_v8(d, w0[0], w0[1], w0[2], w0[3], w0[4], w0[5], w0[6], w0[7]);
                st_global_v8(d + 16, w0[8], w0[9], w0[10], w0[11], w0[12], w0[13], w0[14], w0[15]);
                st_global_v8(d + 64, w1[0], w1[1], w1[2], w1[3], w1[4], w1[5], w1[6], w1[7]);
                st_global_v8(d + 80, w1[8], w1[9], w1[10], w1[11], w1[12], w1[13], w1[14], w1[15]);
              } else {
                uint4* d4 = reinterpret_cast<uint4*>(d);
                uint4* e4 = reinterpret_cast<uint4*>(d + 64);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  d4[i] = make_uint4(w0[4 * i], w0[4 * i + 1], w0[4 * i + 2], w0[4 * i + 3]);
                  e4[i] = make_uint4(w1[4 * i], w1[4 * i + 1], w1[4 * i + 2], w1[4 * i + 3]);
                }
              }
            }
          }
          tile_done = true;
        }
      }
      // the GLU kernel's 128 output columns per tile take the same staged route when they lie in the staged segment
      bool glu_staged = false;
      if constexpr (GLU && !AUX && !PRECISE && BN == 256) {
        const EpiSeg& s0 = p.seg[0];
        glu_staged = p.rm_seg == 0 && out_col_tile >= s0.col_begin && out_col_tile + out_bn <= s0.col_begin + s0.ncols &&
                     (p.nseg == 1 || out_col_tile + out_bn <= p.seg[1].col_begin);
      }
      // Staged GLU tile without mask, bias, statistics, gate or residual (the transitions' SwiGLU): the warp's two 32-column
      // chunks go by as four pieces of 16 columns, the tensor-memory load of the next piece issued before the arithmetic of
      // the current one (a `tcgen05.wait::ld` then finds it done), so that one round trip per tile is exposed instead of two.
      if constexpr (GLU && !AUX && !PRECISE && BN == 256) {
        if (glu_staged && p.col_bias == nullptr && p.row_stats == nullptr && !(p.mask_segs & 1) && p.gate == nullptr &&
            p.resid == nullptr) {
          constexpr int kPieces = 2 * (OUT_BN_GLU / (32 * (kEpiWarps / 4)));   // 16-column pieces of this warp: 4
          uint8_t* buf = s_stage_out + (rm_use & 1) * Cfg::kRowTileBytes;
          auto piece_col = [&](int i) { return chunk_phase * 32 + (i >> 1) * (32 * (kEpiWarps / 4)) + (i & 1) * 16; };
          uint32_t va[16], ga[16], vb[16], gb[16];
          ptx::tmem_ld_32x32b_x16(t_row + piece_col(0), va);
          ptx::tmem_ld_32x32b_x16(t_row + OUT_BN_GLU + piece_col(0), ga);
          const bool swiglu = p.glu != GLU_SIGMOID;
          auto finish_piece = [&](int c, const uint32_t (&vv)[16], const uint32_t (&gg)[16]) {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              const float a0 = __uint_as_float(vv[i]), a1 = __uint_as_float(vv[i + 1]);
              const float g0 = __uint_as_float(gg[i]), g1 = __uint_as_float(gg[i + 1]);
              const float r0 = swiglu ? glu_half(a0, a0) * g0 : glu_half(a0, g0);
              const float r1 = swiglu ? glu_half(a1, a1) * g1 : glu_half(a1, g1);
              w[i >> 1] = pack_bf16x2(r0, r1);
            }
            uint8_t* rowp = buf + (c >> 6) * (Cfg::kRowTileBytes / 2) + r * 128;
            const int piece = (c & 63) >> 3;
            *reinterpret_cast<uint4*>(rowp + (((piece) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4*>(rowp + (((piece + 1) ^ (r & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
          };
#pragma unroll
          for (int i = 0; i < kPieces; i += 2) {
            ptx::tmem_ld_wait();
            if (i + 1 < kPieces) {
              ptx::tmem_ld_32x32b_x16(t_row + piece_col(i + 1), vb);
              ptx::tmem_ld_32x32b_x16(t_row + OUT_BN_GLU + piece_col(i + 1), gb);
            }
            finish_piece(piece_col(i), va, ga);
            ptx::tmem_ld_wait();
            if (i + 2 < kPieces) {
              ptx::tmem_ld_32x32b_x16(t_row + piece_col(i + 2), va);
              ptx::tmem_ld_32x32b_x16(t_row + OUT_BN_GLU + piece_col(i + 2), ga);
            }
            if (i + 1 < kPieces) finish_piece(piece_col(i + 1), vb, gb);
          }
          tile_done = true;
        }
      }
      if (!tile_done)
#pragma unroll 1
      for (int c = chunk_phase * 32; c < out_bn; c += 32 * (kEpiWarps / 4)) {
        const int out_col = out_col_tile + c;
        // Float32 row-major output with gate / residual (the sampler's output projections): a thread owns one row, so its
        // 16-byte accesses to global memory would touch 32 different 128-byte lines per warp instruction.  Instead the warp
        // copies the chunk's gate logits (32 rows x 64 bytes) and residual (32 rows x 128 bytes) into its own shared-memory
        // tile with lane-contiguous asynchronous copies, issued here so that they fly under the tensor-memory load, and
        // writes the result back the same way.  Only warp-level synchronisation is involved.
        bool xp = false;
        uint8_t* xp_res = nullptr;
        uint8_t* xp_gate = nullptr;
        if constexpr (BN == 128 && !GLU && !AUX && !PRECISE) {
          xp = p.xpose != 0 && out_col + 32 <= p.seg[0].ncols;   // uniform across the warp
          if (xp) {
            const EpiSeg& s0 = p.seg[0];
            xp_res = s_stage_out + (warp - 2) * 6144;
            xp_gate = xp_res + 4096;
            const int n_first = nb * kBM + quad * 32;
            if (p.resid != nullptr) {
              const float* rbase = reinterpret_cast<const float*>(p.resid) + static_cast<long long>(b) * s0.s_b +
                                   static_cast<long long>(o) * s0.s_o + out_col;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int rr = i * 4 + (lane >> 3), pc = lane & 7;
                if (n_first + rr < p.n_extent)
                  ptx::cp_async_16(xp_res + rr * 128 + ((pc ^ (rr & 7)) << 4),
                                   rbase + static_cast<long long>(n_first + rr) * s0.s_n + pc * 4);
              }
            }
            if (p.gate != nullptr) {
              const __nv_bfloat16* gbase = p.gate + static_cast<long long>(b) * p.g_b + static_cast<long long>(o) * p.g_o + out_col;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int rr = i * 8 + (lane >> 2), pc = lane & 3;
                if (n_first + rr < p.n_extent)
                  ptx::cp_async_16(xp_gate + rr * 64 + ((pc ^ ((rr >> 1) & 3)) << 4),
                                   gbase + static_cast<long long>(n_first + rr) * p.g_n + pc * 8);
              }
            }
          }
        }
        float v[32];
        if (GLU && !PRECISE) {
          // value and gate columns are fetched together: one round trip to tensor memory per chunk
          uint32_t raw[32], rawg[32];
          ptx::tmem_ld_32x32b_x32(t_row + c, raw);
          ptx::tmem_ld_32x32b_x32(t_row + OUT_BN_GLU + c, rawg);
          ptx::tmem_ld_wait();
          if (p.glu == GLU_SIGMOID) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = glu_half(__uint_as_float(raw[i]), __uint_as_float(rawg[i]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float a = __uint_as_float(raw[i]);   // a / 2
              v[i] = glu_half(a, a) * __uint_as_float(rawg[i]);
            }
          }
        } else {
          {
            uint32_t raw[32];
            ptx::tmem_ld_32x32b_x32(t_row + c, raw);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
            if (PRECISE) {
              ptx::tmem_ld_32x32b_x32(t_row + BN + c, raw);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] += __uint_as_float(raw[i]);
            }
          }
          if (GLU) {
            uint32_t raw[32];
            ptx::tmem_ld_32x32b_x32(t_row + OUT_BN_GLU + c, raw);
            ptx::tmem_ld_wait();
            if (PRECISE) {
              uint32_t raw2[32];
              ptx::tmem_ld_32x32b_x32(t_row + BN + OUT_BN_GLU + c, raw2);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) + __uint_as_float(raw2[i]));
            }
            if (p.glu == GLU_SIGMOID) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                v[i] *= PRECISE ? sigmoidf_exact(__uint_as_float(raw[i])) : sigmoidf_fast(__uint_as_float(raw[i]));
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                v[i] = v[i] * (PRECISE ? sigmoidf_exact(v[i]) : sigmoidf_fast(v[i])) * __uint_as_float(raw[i]);
            }
          }
        }
        // which segment does this chunk belong to
        int si = 0;
        if (p.nseg > 1 && out_col >= p.seg[1].col_begin) si = 1;
        if (p.nseg > 2 && out_col >= p.seg[2].col_begin) si = 2;
        const EpiSeg& sg = p.seg[si];
        const int col_local = out_col - sg.col_begin;
        if (col_local >= sg.ncols) continue;  // uniform across the warp
        if (p.col_bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] += (col_local + i < sg.ncols) ? p.col_bias[out_col + i] : 0.0f;
        }
        if (p.row_stats != nullptr && si == 0) {
          // folded LayerNorm of the A rows: acc was computed on the raw rows with gamma folded into the weights
          const float2 st = row_ok ? p.row_stats[(static_cast<long long>(b) * p.o_extent + o) * p.n_extent + n] : make_float2(0.f, 1.f);
          const float4* s1 = reinterpret_cast<const float4*>(p.col_s1 + out_col);
          const float4* s0 = reinterpret_cast<const float4*>(p.col_s0 + out_col);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 a1 = __ldg(s1 + q), a0 = __ldg(s0 + q);
            v[4 * q] = fmaf(st.y, fmaf(-st.x, a1.x, v[4 * q]), a0.x);
            v[4 * q + 1] = fmaf(st.y, fmaf(-st.x, a1.y, v[4 * q + 1]), a0.y);
            v[4 * q + 2] = fmaf(st.y, fmaf(-st.x, a1.z, v[4 * q + 2]), a0.z);
            v[4 * q + 3] = fmaf(st.y, fmaf(-st.x, a1.w, v[4 * q + 3]), a0.w);
          }
        }
        if ((p.mask_segs >> si) & 1) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] *= mask_v;
        }
        if (sg.tma_slot >= 0) {
          // channel-major segment: the four warps that hold the same 32 columns of the tile (one per TMEM lane
          // quadrant) transpose their pieces into one [32 channels][128 rows] shared-memory slab (two slabs per
          // group, used alternately) and one thread hands it to a TMA store: 32 pieces of 256 contiguous bytes.
          // Rows and channels outside the tensor are clipped by the copy engine.
          const int grp = chunk_phase;
          uint8_t* slab = s_stage_out + (grp * 2 + (staging_use & 1)) * (32 * kBM * 2);
          __nv_bfloat16* col0 = reinterpret_cast<__nv_bfloat16*>(slab) + r;
          const bool issuer = (quad == 0 && lane == 0);
          uint64_t* bar_free = &cm_bar[grp * 2];
          uint64_t* bar_done = &cm_bar[grp * 2 + 1];
          const uint32_t par = staging_use & 1;
          if (issuer) ptx::tma_store_wait_read_le1();  // the store that last read this slab (two uses ago) is done
          ptx::mbar_arrive(bar_free);
          if (!ptx::mbar_wait(bar_free, par, 108)) { ok = false; break; }
          // packed conversions (two values per instruction), then the halves go to their channels' rows
          unsigned short* col0u = reinterpret_cast<unsigned short*>(col0);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint32_t w2 = pack_bf16x2(v[i], v[i + 1]);
            col0u[i * kBM] = static_cast<unsigned short>(w2 & 0xffffu);
            col0u[(i + 1) * kBM] = static_cast<unsigned short>(w2 >> 16);
          }
          ptx::fence_proxy_async_smem();
          ptx::mbar_arrive(bar_done);
          if (issuer) {
            if (!ptx::mbar_wait(bar_done, par, 109)) { ok = false; break; }
            ptx::tma_store_4d(sg.tma_slot == 0 ? &tm_out0 : &tm_out1, slab, nb * kBM, o, col_local, b);
            ptx::tma_store_commit();
          }
          ++staging_use;
          continue;
        }
        const long long row_off = static_cast<long long>(b) * sg.s_b + static_cast<long long>(o) * sg.s_o +
                                  static_cast<long long>(n) * sg.s_n;
        if constexpr (BN == 128 && !GLU && !AUX && !PRECISE) {
          if (xp) {
            const int rl = lane;   // this thread's row within the warp's 32
            ptx::cp_async_wait_all();
            __syncwarp();
            if (p.gate != nullptr) {
              const uint8_t* grow = xp_gate + rl * 64;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 u = *reinterpret_cast<const uint4*>(grow + ((q ^ ((rl >> 1) & 3)) << 4));
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
                  v[q * 8 + j * 2] *= sigmoidf_fast(f.x);
                  v[q * 8 + j * 2 + 1] *= sigmoidf_fast(f.y);
                }
              }
            }
            uint8_t* rrow = xp_res + rl * 128;
            if (p.resid != nullptr) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 f = *reinterpret_cast<const float4*>(rrow + ((q ^ (rl & 7)) << 4));
                v[q * 4] = fmaf(f.x, 1.0f, v[q * 4]); v[q * 4 + 1] = fmaf(f.y, 1.0f, v[q * 4 + 1]);
                v[q * 4 + 2] = fmaf(f.z, 1.0f, v[q * 4 + 2]); v[q * 4 + 3] = fmaf(f.w, 1.0f, v[q * 4 + 3]);
              }
            }
            // every thread writes its own row; below, eight lanes share a row
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<float4*>(rrow + ((q ^ (rl & 7)) << 4)) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
            __syncwarp();
            {
              const int n_first = nb * kBM + quad * 32;
              float* obase = reinterpret_cast<float*>(sg.dst) + static_cast<long long>(b) * sg.s_b +
                             static_cast<long long>(o) * sg.s_o + col_local;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int rr = i * 4 + (lane >> 3), pc = lane & 7;
                const float4 f = *reinterpret_cast<const float4*>(xp_res + rr * 128 + ((pc ^ (rr & 7)) << 4));
                if (n_first + rr < p.n_extent)
                  *reinterpret_cast<float4*>(obase + static_cast<long long>(n_first + rr) * sg.s_n + pc * 4) = f;
              }
            }
            __syncwarp();   // the tile is free for the next chunk's copies
            continue;
          }
        }
        if (AUX && si == 0) {
          // gate logits and residual come from the tiles the producer prefetched (128-byte swizzled rows)
          const uint8_t* rowp = aux_tile + (c >> 6) * (kBM * 128) + r * 128;
          const int cbase = ((c >> 5) & 1) * 4;
          if (p.aux_gate) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 u = *reinterpret_cast<const uint4*>(rowp + (((cbase + q) ^ (r & 7)) << 4));
              const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                v[q * 8 + j * 2] *= sigmoidf_fast(__uint_as_float(w[j] << 16));
                v[q * 8 + j * 2 + 1] *= sigmoidf_fast(__uint_as_float(w[j] & 0xffff0000u));
              }
            }
          }
          if (p.aux_resid) {
            const uint8_t* rrow = rowp + Cfg::kAuxTileBytes;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 u = *reinterpret_cast<const uint4*>(rrow + (((cbase + q) ^ (r & 7)) << 4));
              const uint32_t w[4] = {u.x, u.y, u.z, u.w};
              if (p.resid_scale != nullptr) {
                const float4 s0 = __ldg(reinterpret_cast<const float4*>(p.resid_scale + out_col + q * 8));
                const float4 s1 = __ldg(reinterpret_cast<const float4*>(p.resid_scale + out_col + q * 8 + 4));
                const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  v[q * 8 + j * 2] = fmaf(__uint_as_float(w[j] << 16), sc[j * 2], v[q * 8 + j * 2]);
                  v[q * 8 + j * 2 + 1] = fmaf(__uint_as_float(w[j] & 0xffff0000u), sc[j * 2 + 1], v[q * 8 + j * 2 + 1]);
                }
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  v[q * 8 + j * 2] += __uint_as_float(w[j] << 16);
                  v[q * 8 + j * 2 + 1] += __uint_as_float(w[j] & 0xffff0000u);
                }
              }
            }
          }
        } else if (!AUX && si == 0 && row_ok) {
          if (PRECISE && p.gate != nullptr) {
            const float* g = reinterpret_cast<const float*>(p.gate) + static_cast<long long>(b) * p.g_b +
                             static_cast<long long>(o) * p.g_o + static_cast<long long>(n) * p.g_n +
                             static_cast<long long>(col_local) * p.g_col;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col_local + i < sg.ncols) v[i] *= sigmoidf_exact(g[static_cast<long long>(i) * p.g_col]);
          } else if (p.gate != nullptr) {
            const __nv_bfloat16* g = p.gate + static_cast<long long>(b) * p.g_b + static_cast<long long>(o) * p.g_o +
                                     static_cast<long long>(n) * p.g_n + static_cast<long long>(col_local) * p.g_col;
            if (p.g_col == 1 && col_local + 32 <= sg.ncols) {
              const uint4* g4 = reinterpret_cast<const uint4*>(g);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 u = g4[q];
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
                  v[q * 8 + j * 2] *= sigmoidf_fast(f.x);
                  v[q * 8 + j * 2 + 1] *= sigmoidf_fast(f.y);
                }
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col_local + i < sg.ncols) v[i] *= sigmoidf_fast(__bfloat162float(g[static_cast<long long>(i) * p.g_col]));
            }
          }
          if (p.resid != nullptr && sg.vec && col_local + 32 <= sg.ncols) {
            if (sg.out_fp32) {
              const float4* rs = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.resid) + row_off + col_local);
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 f = rs[q];
                const float4 sc = p.resid_scale != nullptr ? __ldg(reinterpret_cast<const float4*>(p.resid_scale + out_col + q * 4))
                                                           : make_float4(1.f, 1.f, 1.f, 1.f);
                v[q * 4] = fmaf(f.x, sc.x, v[q * 4]); v[q * 4 + 1] = fmaf(f.y, sc.y, v[q * 4 + 1]);
                v[q * 4 + 2] = fmaf(f.z, sc.z, v[q * 4 + 2]); v[q * 4 + 3] = fmaf(f.w, sc.w, v[q * 4 + 3]);
              }
            } else {
              const uint4* rs = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.resid) + row_off + col_local);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 u = rs[q];
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
                  const float sx = p.resid_scale != nullptr ? __ldg(p.resid_scale + out_col + q * 8 + j * 2) : 1.0f;
                  const float sy = p.resid_scale != nullptr ? __ldg(p.resid_scale + out_col + q * 8 + j * 2 + 1) : 1.0f;
                  v[q * 8 + j * 2] = fmaf(f.x, sx, v[q * 8 + j * 2]);
                  v[q * 8 + j * 2 + 1] = fmaf(f.y, sy, v[q * 8 + j * 2 + 1]);
                }
              }
            }
          } else if (p.resid != nullptr) {
            if (sg.out_fp32) {
              const float* rs = reinterpret_cast<const float*>(p.resid) + row_off + static_cast<long long>(col_local) * sg.s_col;
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col_local + i < sg.ncols)
                  v[i] = fmaf(rs[static_cast<long long>(i) * sg.s_col], p.resid_scale != nullptr ? p.resid_scale[out_col + i] : 1.0f, v[i]);
            } else {
              const __nv_bfloat16* rs =
                  reinterpret_cast<const __nv_bfloat16*>(p.resid) + row_off + static_cast<long long>(col_local) * sg.s_col;
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col_local + i < sg.ncols)
                  v[i] = fmaf(__bfloat162float(rs[static_cast<long long>(i) * sg.s_col]),
                              p.resid_scale != nullptr ? p.resid_scale[out_col + i] : 1.0f, v[i]);
            }
          }
        }
        if constexpr (GLU && !AUX && !PRECISE && BN == 256) {
          if (glu_staged) {
            uint8_t* rowp = s_stage_out + (rm_use & 1) * Cfg::kRowTileBytes + (c >> 6) * (Cfg::kRowTileBytes / 2) + r * 128;
            const int piece = (c & 63) >> 3;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
              *reinterpret_cast<uint4*>(rowp + (((piece + q4) ^ (r & 7)) << 4)) =
                  make_uint4(pack_bf16x2(v[8 * q4], v[8 * q4 + 1]), pack_bf16x2(v[8 * q4 + 2], v[8 * q4 + 3]),
                             pack_bf16x2(v[8 * q4 + 4], v[8 * q4 + 5]), pack_bf16x2(v[8 * q4 + 6], v[8 * q4 + 7]));
            continue;
          }
        }
        if (PRECISE && sg.split)
          epi_store_split(sg, row_off, col_local, v, row_ok);
        else
          epi_store_chunk(sg, row_off, col_local, v, row_ok);
      }
      if constexpr (GLU && !AUX && !PRECISE && BN == 256) {
        if (glu_staged && ok) {
          ptx::fence_proxy_async_smem();
          const bool issuer = (quad == 0 && chunk_phase == 0 && lane == 0);
          if (issuer) ptx::tma_store_wait_read();
          ptx::mbar_arrive(&rm_bar[rm_use & 1]);
          if (!ptx::mbar_wait(&rm_bar[rm_use & 1], (rm_use >> 1) & 1, 112)) {
            ok = false;
          } else if (issuer) {
            const uint8_t* buf = s_stage_out + (rm_use & 1) * Cfg::kRowTileBytes;
            const int col0 = out_col_tile - p.seg[0].col_begin;
            ptx::tma_store_4d(&tm_out0, buf, col0, nb * kBM, o, b);
            ptx::tma_store_4d(&tm_out0, buf + Cfg::kRowTileBytes / 2, col0 + 64, nb * kBM, o, b);
            ptx::tma_store_commit();
          }
          ++rm_use;
        }
      }
      }
      if (!ok) break;
      if (AUX) {
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&aux_empty[tile_iter & 1]);
      }
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&tmem_empty[acc]);
      if (threadIdx.x == 64) KFB_GSTAMP(4 + tile_iter * 4 + 1);
    }
    if (quad == 0 && lane == 0) ptx::tma_store_wait_all();
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) KFB_GSTAMP(1);
#undef KFB_GSTAMP
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, PRECISE ? 2 * Cfg::kTmemCols : Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
struct GemmOperandA {  // A[(b,o,n), k], strides in elements
  const void* ptr;
  long long s_n, s_o, s_b;
  long long s_k = 0;       // != 0: K-outer storage, element (row, k) at ptr + k * s_k + row (rows contiguous, s_n = 1):
                           // the operand is then read MN-major (n_extent must cover whole 64-row boxes in memory)
  int k_inner = 0;         // != 0 (set on both operands alike): K lies in pieces of k_inner contiguous elements, piece h of a
  long long s_k_hi = 0;    // row starting s_k_hi * h elements after piece 0
};
struct GemmOperandB {  // B[(b), col, k]; optionally col = hi * col_inner + lo with its own stride for hi
  const void* ptr;
  long long s_col, s_b;
  int col_inner = 0;       // 0: plain rows
  long long s_col_hi = 0;
  int k_inner = 0;         // as for GemmOperandA
  long long s_k_hi = 0;
};

// Fills the tile bookkeeping of `p`, builds the tensor maps and launches on `stream`.
// `tag` names the launch in the profile report (a string literal).
// A segment whose rows are contiguous along n (s_n == 1) and whose other strides and base are 16-byte
// aligned can go through the TMA-store path; the launcher decides and fills `tma_slot`.
int launch_gemm_bf16(cudaStream_t stream, const GemmOperandA& a, const GemmOperandB& b, GemmParams p, int force_bn = 0,
                     const char* tag = "gemm");

// Debugging aid: launches whose tag equals `tag` store per-tile clock stamps of CTA 0 into `device_buffer`
// (>= 512 long longs); nullptr switches it off.
void set_gemm_trace(long long* device_buffer, const char* tag);

}  // namespace kfb
