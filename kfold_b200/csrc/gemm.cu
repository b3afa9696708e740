// Host launcher of the persistent tcgen05 GEMM (see gemm.cuh for the kernel).
#include <limits.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "gemm.cuh"

namespace kfb {

template <int BN, bool GLU, bool AUX, bool PRECISE, bool SWAP = false>
static int launch_variant(cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap* tout,
                          const GemmParams& p, const char* tag) {
  using Cfg = GemmCfg<BN>;
  static std::once_flag once[64];
  int dev = 0;
  KFB_CUDA(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  std::call_once(once[dev & 63], [&] {
    attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<BN, GLU, AUX, PRECISE, SWAP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::kSmemBytes);
  });
  KFB_CUDA(attr_err);
  const int total = p.num_m_tiles * p.num_n_tiles;
  const int grid = total < sm_count() ? total : sm_count();
  GemmParams q = p;
  {
    // the persistent loops step by the grid size: its digits in the (n tile, row block, outer, batch) index
    const int m_step = grid / q.num_n_tiles;
    q.step_n_tile = grid - m_step * q.num_n_tiles;
    q.step_nb = m_step % q.n_blocks;
    const int rest = m_step / q.n_blocks;
    q.step_o = rest % q.o_extent;
    q.step_b = rest / q.o_extent;
  }
  {
    LaunchScope scope(stream, tag);
    gemm_bf16_kernel<BN, GLU, AUX, PRECISE, SWAP><<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(ta, tb, tout[0], tout[1], q);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

template <int BN>
static int launch_bn(cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap* tout,
                     GemmParams p, const char* tag) {
  using Cfg = GemmCfg<BN>;
  if (p.aux && Cfg::stages_for(Cfg::kAuxBytes) < 2) p.aux = 0;  // no room (BN = 256): fall back to direct loads
  p.stages = Cfg::stages_for(p.aux ? Cfg::kAuxBytes : Cfg::kStagingBytes);
  if constexpr (BN <= 128) {
    if (p.precise) {
      p.k_main_blocks = (p.k_extent / 6) / kBK;
      if (p.k_main_blocks == 0) p.k_main_blocks = 1;  // short K: the first block mixes parts, harmless
      if (p.glu) return launch_variant<BN, true, false, true>(stream, ta, tb, tout, p, tag);
      return launch_variant<BN, false, false, true>(stream, ta, tb, tout, p, tag);
    }
  }
  if constexpr (BN == 256) {
    if (p.glu && p.swap) {
      p.stages = Cfg::stages_for(Cfg::kSwapStagingBytes);
      return launch_variant<BN, true, false, false, true>(stream, ta, tb, tout, p, tag);
    }
  }
  if (p.glu) {
    p.stages = Cfg::stages_for(Cfg::kGluStagingBytes);
    return launch_variant<BN, true, false, false>(stream, ta, tb, tout, p, tag);
  }
  if constexpr (BN <= 128) {
    if (p.aux) return launch_variant<BN, false, true, false>(stream, ta, tb, tout, p, tag);
  }
  return launch_variant<BN, false, false, false>(stream, ta, tb, tout, p, tag);
}

static long long* g_trace_buf = nullptr;
static char g_trace_tag[64] = "";
void set_gemm_trace(long long* device_buffer, const char* tag) {
  g_trace_buf = device_buffer;
  snprintf(g_trace_tag, sizeof(g_trace_tag), "%s", tag ? tag : "");
}

int launch_gemm_bf16(cudaStream_t stream, const GemmOperandA& a, const GemmOperandB& b, GemmParams p, int force_bn,
                     const char* tag) {
  KFB_CHECK_ARG(p.n_extent > 0 && p.o_extent > 0 && p.batch > 0 && p.n_cols > 0 && p.k_extent > 0, "empty GEMM");
  KFB_CHECK_ARG(p.nseg >= 1 && p.nseg <= 3, "GEMM needs 1..3 output segments");
  int bn = force_bn;
  if (bn == 0) bn = p.n_cols >= 256 ? 256 : (p.n_cols > 64 ? 128 : 64);
  if (p.precise && bn > 128) bn = 128;  // the fp32-accurate variant keeps four accumulators in tensor memory
  // One row-major float32 segment with a gate and / or a residual (the output projections of the sampler's float32 activation
  // stream): 128-column tiles whose epilogue moves gate, residual and output through per-warp shared-memory tiles.
  p.xpose = 0;
  if (!p.precise && !p.glu && force_bn == 0 && bn >= 128 && p.nseg == 1 && a.s_k == 0 && a.k_inner == 0 && b.col_inner == 0 &&
      (p.gate != nullptr || p.resid != nullptr) && p.resid_scale == nullptr) {
    const EpiSeg& sg = p.seg[0];
    const bool seg_ok = sg.out_fp32 && sg.vec && sg.s_col == 1 && sg.col_begin == 0 && !sg.split && sg.ncols % 32 == 0 &&
                        sg.s_n % 4 == 0 && sg.s_o % 4 == 0 && sg.s_b % 4 == 0 &&
                        (p.resid == nullptr || (reinterpret_cast<uintptr_t>(p.resid) & 15) == 0);
    const bool gate_ok = p.gate == nullptr ||
                         (p.g_col == 1 && (reinterpret_cast<uintptr_t>(p.gate) & 15) == 0 && p.g_n % 8 == 0 && p.g_o % 8 == 0 &&
                          p.g_b % 8 == 0);
    if (seg_ok && gate_ok) {
      p.xpose = 1;
      bn = 128;
    }
  }
  KFB_CHECK_ARG(bn == 64 || bn == 128 || bn == 256, "unsupported BN %d", bn);
  if (p.precise) KFB_CHECK_ARG(p.k_extent % 6 == 0, "precise GEMM: K=%d is not six equal parts", p.k_extent);
  if (p.glu) KFB_CHECK_ARG(p.n_cols % bn == 0, "GLU GEMM needs n_cols (%d) to be a multiple of the N tile (%d)", p.n_cols, bn);
  for (int i = 0; i < p.nseg; ++i) KFB_CHECK_ARG(p.seg[i].col_begin % 32 == 0, "segment start must be a multiple of 32");
  p.trace = (g_trace_buf != nullptr && strcmp(g_trace_tag, tag) == 0) ? g_trace_buf : nullptr;
  p.n_blocks = cdiv(p.n_extent, kBM);
  p.num_m_tiles = p.n_blocks * p.o_extent * p.batch;
  p.num_n_tiles = cdiv(p.n_cols, bn);

  CUtensorMap ta, tb;
  p.a_mn_major = a.s_k != 0 ? 1 : 0;
  p.k_inner = a.k_inner;
  KFB_CHECK_ARG(a.k_inner == b.k_inner, "split K: both operands must be split alike (%d, %d)", a.k_inner, b.k_inner);
  if (p.k_inner) {
    KFB_CHECK_ARG(!p.a_mn_major && !p.precise && p.k_inner % kBK == 0 && p.k_extent % p.k_inner == 0,
                  "split K: pieces of %d elements (multiple of %d) in K=%d, plain bf16 GEMM", p.k_inner, kBK, p.k_extent);
    const uint64_t dims[5] = {(uint64_t)p.k_inner, (uint64_t)p.n_extent, (uint64_t)p.o_extent, (uint64_t)(p.k_extent / p.k_inner),
                              (uint64_t)p.batch};
    const uint64_t str[4] = {(uint64_t)a.s_n * 2, (uint64_t)a.s_o * 2, (uint64_t)a.s_k_hi * 2, (uint64_t)a.s_b * 2};
    const uint32_t box[5] = {kBK, kBM, 1, 1, 1};
    KFB_TRY(make_tmap(&ta, a.ptr, 2, 5, dims, str, box, 128));
  } else if (p.a_mn_major) {
    KFB_CHECK_ARG(a.s_n == 1 && p.k_extent % kBK == 0 && !p.precise && !p.glu, "K-outer A operand: rows must be contiguous, K a "
                  "multiple of %d, plain bf16 GEMM", kBK);
    const uint64_t dims[4] = {(uint64_t)p.n_extent, (uint64_t)p.k_extent, (uint64_t)p.o_extent, (uint64_t)p.batch};
    const uint64_t str[3] = {(uint64_t)a.s_k * 2, (uint64_t)a.s_o * 2, (uint64_t)a.s_b * 2};
    const uint32_t box[4] = {64, kBK, 1, 1};
    KFB_TRY(make_tmap(&ta, a.ptr, 2, 4, dims, str, box, 128));
  } else {
    const uint64_t dims[4] = {(uint64_t)p.k_extent, (uint64_t)p.n_extent, (uint64_t)p.o_extent, (uint64_t)p.batch};
    const uint64_t str[3] = {(uint64_t)a.s_n * 2, (uint64_t)a.s_o * 2, (uint64_t)a.s_b * 2};
    const uint32_t box[4] = {kBK, kBM, 1, 1};
    KFB_TRY(make_tmap(&ta, a.ptr, 2, 4, dims, str, box, 128));
  }
  {
    const int inner = b.col_inner > 0 ? b.col_inner : p.n_cols;
    if (b.col_inner > 0)
      KFB_CHECK_ARG(p.n_cols % inner == 0 && inner % bn == 0, "split B operand: %d columns in pieces of %d, tile %d", p.n_cols,
                    inner, bn);
    p.b_col_inner = inner;
    if (p.k_inner) {
      const uint64_t dims[5] = {(uint64_t)p.k_inner, (uint64_t)inner, (uint64_t)(p.n_cols / inner),
                                (uint64_t)(p.k_extent / p.k_inner), (uint64_t)(p.b_batched ? p.batch : 1)};
      const uint64_t str[4] = {(uint64_t)b.s_col * 2, (uint64_t)b.s_col_hi * 2, (uint64_t)b.s_k_hi * 2, (uint64_t)b.s_b * 2};
      const uint32_t box[5] = {kBK, (uint32_t)bn, 1, 1, 1};
      KFB_TRY(make_tmap(&tb, b.ptr, 2, 5, dims, str, box, 128));
    } else {
    const uint64_t dims[4] = {(uint64_t)p.k_extent, (uint64_t)inner, (uint64_t)(p.n_cols / inner),
                              (uint64_t)(p.b_batched ? p.batch : 1)};
    const uint64_t str[3] = {(uint64_t)b.s_col * 2, (uint64_t)b.s_col_hi * 2, (uint64_t)b.s_b * 2};
    const uint32_t box[4] = {kBK, (uint32_t)bn, 1, 1};
    KFB_TRY(make_tmap(&tb, b.ptr, 2, 4, dims, str, box, 128));
    }
  }
  // channel-major bf16 segments that satisfy the TMA alignment rules are stored through shared memory
  CUtensorMap tout[2];
  tout[0] = ta;  // placeholders (never dereferenced unless a segment selects them)
  tout[1] = ta;
  int next_slot = 0;
  // a sigmoid-GLU GEMM whose only output is channel-major bf16 is computed in the swapped orientation
  p.swap = (p.glu == GLU_SIGMOID && bn == 256 && p.nseg == 1 && !p.precise && p.seg[0].s_n == 1 && p.seg[0].s_col != 1 &&
            !p.seg[0].out_fp32 && p.seg[0].col_begin == 0 && p.n_cols % 256 == 0 && p.col_bias == nullptr &&
            p.gate == nullptr && p.resid == nullptr && (p.rowmask == nullptr || (p.mask_segs & 1)))
               ? 1 : 0;
  // ... and, when the destination satisfies the copy engine's alignment rules, stored as whole tiles by TMA
  p.swap_staged = 0;
  if (p.swap) {
    const EpiSeg& sg = p.seg[0];
    const bool aligned = (reinterpret_cast<uintptr_t>(sg.dst) & 15) == 0 && sg.s_col % 8 == 0 &&
                         (sg.s_o % 8 == 0 && (sg.s_o != 0 || p.o_extent == 1)) && (sg.s_b % 8 == 0 && (sg.s_b != 0 || p.batch == 1));
    if (aligned) {
      const uint64_t dims[4] = {(uint64_t)p.n_extent, (uint64_t)p.o_extent, (uint64_t)sg.ncols, (uint64_t)p.batch};
      const uint64_t str[3] = {(uint64_t)sg.s_o * 2, (uint64_t)sg.s_col * 2, (uint64_t)sg.s_b * 2};
      const uint32_t box[4] = {64, 1, kBM, 1};
      KFB_TRY(make_tmap(&tout[0], sg.dst, 2, 4, dims, str, box, 128));
      p.swap_staged = 1;
      next_slot = 1;
    }
  }
  // trailing channel-major bf16 segments that start on a tile boundary are computed in the swapped orientation as well
  // (plain BN = 128 kernel): the threads then store runs of consecutive positions directly
  p.swap_col_begin = INT_MAX;
  if (bn == 128 && !p.glu && !p.precise && !p.a_mn_major) {
    for (int i = p.nseg - 1; i >= 0; --i) {
      const EpiSeg& sg = p.seg[i];
      const bool cm = sg.s_n == 1 && sg.s_col != 1 && !sg.out_fp32 && !sg.split && sg.col_begin % 128 == 0 &&
                      !((p.mask_segs >> i) & 1) && (i > 0 || (p.gate == nullptr && p.resid == nullptr));
      if (!cm) break;
      p.swap_col_begin = sg.col_begin;
    }
  }
  for (int i = 0; i < p.nseg; ++i) {
    EpiSeg& sg = p.seg[i];
    sg.tma_slot = -1;
    if (p.swap || sg.col_begin >= p.swap_col_begin) continue;
    const bool aligned = (reinterpret_cast<uintptr_t>(sg.dst) & 15) == 0 && sg.s_o % 8 == 0 && sg.s_col % 8 == 0 &&
                         (sg.s_b % 8 == 0 || p.batch == 1) && (sg.s_o != 0 || p.o_extent == 1);
    if (sg.s_n == 1 && sg.s_col != 1 && !sg.out_fp32 && aligned && next_slot < 2 && !p.precise) {
      const uint64_t dims[4] = {(uint64_t)p.n_extent, (uint64_t)p.o_extent, (uint64_t)sg.ncols, (uint64_t)p.batch};
      const uint64_t str[3] = {(uint64_t)sg.s_o * 2, (uint64_t)sg.s_col * 2, (uint64_t)sg.s_b * 2};
      const uint32_t box[4] = {kBM, 1, 32, 1};
      KFB_TRY(make_tmap(&tout[next_slot], sg.dst, 2, 4, dims, str, box, 0));
      sg.tma_slot = next_slot++;
    }
  }
  // gate / residual prefetch: only without staged segments, bf16 tensors, full 32-column chunks, aligned strides
  p.aux = 0;
  p.aux_gate = 0;
  p.aux_resid = 0;
  if (!p.precise && !p.xpose && next_slot == 0 && p.nseg == 1 && p.seg[0].vec && (p.gate != nullptr || p.resid != nullptr) &&
      bn >= 64 && p.n_cols % 32 == 0 && !p.glu) {
    const EpiSeg& sg = p.seg[0];
    bool ok_g = true, ok_r = true;
    if (p.gate != nullptr)
      ok_g = p.g_col == 1 && (reinterpret_cast<uintptr_t>(p.gate) & 15) == 0 && p.g_n % 8 == 0 && p.g_n != 0 &&
             p.g_o % 8 == 0 && (p.g_o != 0 || p.o_extent == 1) && p.g_b % 8 == 0 && (p.g_b != 0 || p.batch == 1);
    if (p.resid != nullptr)
      ok_r = !sg.out_fp32 && (reinterpret_cast<uintptr_t>(p.resid) & 15) == 0 && sg.s_n % 8 == 0 && sg.s_o % 8 == 0 &&
             (sg.s_o != 0 || p.o_extent == 1) && sg.s_b % 8 == 0 && (sg.s_b != 0 || p.batch == 1);
    if (ok_g && ok_r) {
      const uint32_t box[4] = {64, kBM, 1, 1};
      const uint64_t dims[4] = {(uint64_t)p.n_cols, (uint64_t)p.n_extent, (uint64_t)p.o_extent, (uint64_t)p.batch};
      if (p.gate != nullptr) {
        const uint64_t str[3] = {(uint64_t)p.g_n * 2, (uint64_t)p.g_o * 2, (uint64_t)p.g_b * 2};
        KFB_TRY(make_tmap(&tout[0], p.gate, 2, 4, dims, str, box, 128));
        p.aux_gate = 1;
      }
      if (p.resid != nullptr) {
        const uint64_t str[3] = {(uint64_t)sg.s_n * 2, (uint64_t)sg.s_o * 2, (uint64_t)sg.s_b * 2};
        KFB_TRY(make_tmap(&tout[1], p.resid, 2, 4, dims, str, box, 128));
        p.aux_resid = 1;
      }
      p.aux = 1;
    }
  }
  // full tiles of one row-major bf16 segment of the plain BN = 128 kernel leave through shared memory and a TMA store
  p.rm_seg = -1;
  p.rm_slot = 0;
  const bool rm_plain = bn == 128 && !p.glu;
  const bool rm_glu = bn == 256 && p.glu && !p.swap;      // the GLU kernel: 128 output columns per tile
  if ((rm_plain || rm_glu) && !p.precise && !p.aux && !p.a_mn_major && next_slot == 0) {
    for (int i = 0; i < p.nseg; ++i) {
      const EpiSeg& sg = p.seg[i];
      if (rm_glu && (i != 0 || sg.ncols % 128 != 0)) break;   // the GLU route handles segment 0 made of whole tiles only
      const bool ok_seg = sg.s_col == 1 && sg.vec && !sg.out_fp32 && sg.col_begin % 128 == 0 && sg.ncols >= 128 &&
                          sg.col_begin < p.swap_col_begin && (reinterpret_cast<uintptr_t>(sg.dst) & 15) == 0 && sg.s_n % 8 == 0 &&
                          (sg.s_o % 8 == 0 && (sg.s_o != 0 || p.o_extent == 1)) && (sg.s_b % 8 == 0 && (sg.s_b != 0 || p.batch == 1)) &&
                          !((p.mask_segs >> i) & 1) && (i != 0 || (p.gate == nullptr && p.resid == nullptr));
      if (!ok_seg) continue;
      const uint64_t dims[4] = {(uint64_t)sg.ncols, (uint64_t)p.n_extent, (uint64_t)p.o_extent, (uint64_t)p.batch};
      const uint64_t str[3] = {(uint64_t)sg.s_n * 2, (uint64_t)sg.s_o * 2, (uint64_t)sg.s_b * 2};
      const uint32_t box[4] = {64, kBM, 1, 1};
      KFB_TRY(make_tmap(&tout[0], sg.dst, 2, 4, dims, str, box, 128));
      p.rm_seg = i;
      break;
    }
  }
  switch (bn) {
    case 64: return launch_bn<64>(stream, ta, tb, tout, p, tag);
    case 128: return launch_bn<128>(stream, ta, tb, tout, p, tag);
    default: return launch_bn<256>(stream, ta, tb, tout, p, tag);
  }
}

}  // namespace kfb
