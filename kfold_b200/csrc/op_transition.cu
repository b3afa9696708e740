// Transition (LayerNorm -> SwiGLU -> output projection) as a kernel sequence.
//   1. LayerNorm                         x -> xn (bf16)                              [HBM bound]
//   2. GEMM xn [Wa ; Wb]^T with the SwiGLU epilogue  h = silu(u_a) * u_b  (bf16)     [tcgen05]
//   3. GEMM h W_out^T (+ optional residual)                                          [tcgen05]
#include "ops_common.cuh"

using namespace kfb;

namespace {
struct TransWs {
  __nv_bfloat16 *xn, *h;
};
size_t carve(TransWs& w, void* base, long long rows, int c, int hidden) {
  Carver cv(base);
  w.xn = cv.take<__nv_bfloat16>(static_cast<size_t>(rows) * c);
  w.h = cv.take<__nv_bfloat16>(static_cast<size_t>(rows) * hidden);
  return cv.off;
}
}  // namespace

extern "C" {

KFB_API size_t kfb_transition_workspace_bytes(long long rows, int c, int hidden) {
  TransWs w;
  return carve(w, nullptr, rows, c, hidden);
}

KFB_API int kfb_transition_fwd(const void* x, const float* ln_w, const float* ln_b, const void* w_swiglu_packed,
                               const void* w_out, void* out, const void* resid, void* workspace, size_t workspace_bytes,
                               long long rows, int c, int hidden, float eps, int dtype, void* stream_) {
  KFB_CHECK_ARG(x && w_swiglu_packed && w_out && out && workspace, "transition: null pointer");
  KFB_CHECK_ARG(is_dtype(dtype), "transition: bad dtype %d", dtype);
  KFB_CHECK_ARG(rows >= 1 && rows < (1ll << 31), "transition: rows %lld", rows);
  KFB_CHECK_ARG(c % 8 == 0 && hidden % 128 == 0, "transition: c=%d (multiple of 8), hidden=%d (multiple of 128)", c, hidden);
  TransWs w;
  const size_t need = carve(w, workspace, rows, c, hidden);
  KFB_CHECK_ARG(workspace_bytes >= need, "transition: workspace %zu < %zu bytes", workspace_bytes, need);
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "transition: workspace must be 256-byte aligned");
  cudaStream_t stream = as_stream(stream_);
  KFB_TRY(launch_layernorm(stream, x, w.xn, ln_w, ln_b, rows, c, c, c, eps, dtype, KFB_BF16));
  {
    GemmParams p = {};
    p.n_extent = static_cast<int>(rows);
    p.o_extent = 1;
    p.batch = 1;
    p.n_cols = 2 * hidden;
    p.k_extent = c;
    p.glu = GLU_SWIGLU;
    p.nseg = 1;
    p.seg[0] = row_major_seg(w.h, hidden, hidden, 0, 0, 0);
    GemmOperandA a = {w.xn, c, 0, 0};
    GemmOperandB b = {w_swiglu_packed, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 256, "transition_swiglu"));
  }
  {
    GemmParams p = {};
    p.n_extent = static_cast<int>(rows);
    p.o_extent = 1;
    p.batch = 1;
    p.n_cols = c;
    p.k_extent = hidden;
    p.nseg = 1;
    p.seg[0] = row_major_seg(out, c, c, 0, 0, dtype == KFB_FP32);
    p.resid = resid;
    GemmOperandA a = {w.h, hidden, 0, 0};
    GemmOperandB b = {w_out, hidden, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "transition_out"));
  }
  return KFB_OK;
}

}  // extern "C"
