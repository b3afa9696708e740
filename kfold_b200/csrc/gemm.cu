// Host launcher of the persistent tcgen05 GEMM (see gemm.cuh for the kernel).
#include <mutex>

#include "common.cuh"
#include "gemm.cuh"

namespace kfb {

template <int BN>
static int launch_bn(cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, const char* tag) {
  using Cfg = GemmCfg<BN>;
  static std::once_flag once[64];
  int dev = 0;
  KFB_CUDA(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  std::call_once(once[dev & 63], [&] {
    attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  });
  KFB_CUDA(attr_err);
  const int total = p.num_m_tiles * p.num_n_tiles;
  const int grid = total < sm_count() ? total : sm_count();
  {
    LaunchScope scope(stream, tag);
    gemm_bf16_kernel<BN><<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(ta, tb, p);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

int launch_gemm_bf16(cudaStream_t stream, const GemmOperandA& a, const GemmOperandB& b, GemmParams p, int force_bn,
                     const char* tag) {
  KFB_CHECK_ARG(p.n_extent > 0 && p.o_extent > 0 && p.batch > 0 && p.n_cols > 0 && p.k_extent > 0, "empty GEMM");
  KFB_CHECK_ARG(p.nseg >= 1 && p.nseg <= 3, "GEMM needs 1..3 output segments");
  int bn = force_bn;
  if (bn == 0) bn = p.n_cols >= 256 ? 256 : (p.n_cols > 64 ? 128 : 64);
  KFB_CHECK_ARG(bn == 64 || bn == 128 || bn == 256, "unsupported BN %d", bn);
  if (p.glu) KFB_CHECK_ARG(p.n_cols % bn == 0, "GLU GEMM needs n_cols (%d) to be a multiple of the N tile (%d)", p.n_cols, bn);
  for (int i = 0; i < p.nseg; ++i) KFB_CHECK_ARG(p.seg[i].col_begin % 32 == 0, "segment start must be a multiple of 32");
  p.n_blocks = cdiv(p.n_extent, kBM);
  p.num_m_tiles = p.n_blocks * p.o_extent * p.batch;
  p.num_n_tiles = cdiv(p.n_cols, bn);
  if (p.alpha == 0.0f) p.alpha = 1.0f;

  CUtensorMap ta, tb;
  {
    const uint64_t dims[4] = {(uint64_t)p.k_extent, (uint64_t)p.n_extent, (uint64_t)p.o_extent, (uint64_t)p.batch};
    const uint64_t str[3] = {(uint64_t)a.s_n * 2, (uint64_t)a.s_o * 2, (uint64_t)a.s_b * 2};
    const uint32_t box[4] = {kBK, kBM, 1, 1};
    KFB_TRY(make_tmap(&ta, a.ptr, 2, 4, dims, str, box, 128));
  }
  {
    const uint64_t dims[3] = {(uint64_t)p.k_extent, (uint64_t)p.n_cols, (uint64_t)(p.b_batched ? p.batch : 1)};
    const uint64_t str[2] = {(uint64_t)b.s_col * 2, (uint64_t)b.s_b * 2};
    const uint32_t box[3] = {kBK, (uint32_t)bn, 1};
    KFB_TRY(make_tmap(&tb, b.ptr, 2, 3, dims, str, box, 128));
  }
  switch (bn) {
    case 64: return launch_bn<64>(stream, ta, tb, p, tag);
    case 128: return launch_bn<128>(stream, ta, tb, p, tag);
    default: return launch_bn<256>(stream, ta, tb, p, tag);
  }
}

}  // namespace kfb
