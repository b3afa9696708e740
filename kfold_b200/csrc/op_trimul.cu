// Triangle multiplication (outgoing / incoming) as a sequence of sm_100a kernels.
//
//   1. LayerNorm_in                      x -> xn (bf16, position-major)             [HBM bound]
//   2. input projection + gate + mask    ab[ch] = (xn Wp^T) * sigmoid(xn Wg^T) * m  [tcgen05 GEMM, GLU epilogue,
//                                        stored CHANNEL-major so each channel is      channel-major store]
//                                        a dense N x N matrix
//   3. output gate logits                gl = xn Wg_out^T                            [tcgen05 GEMM]
//   4. triangle contraction              t[ch] = A_ch * B_ch^T, batch over channels   [tcgen05 batched GEMM]
//   5. LayerNorm_out, channel-major in   t -> tn (bf16, position-major)             [HBM bound]
//   6. output projection * sigmoid(gl)   out = (tn Wp_out^T) * sigmoid(gl) (+ resid) [tcgen05 GEMM, gated epilogue]
//
// The incoming direction needs t[i,j] = sum_k a[k,i] b[k,j].  Instead of a second,
// MN-major contraction kernel, step 2 walks the pair tensor transposed (the TMA map
// of xn swaps its two position strides) so that it writes a^T and b^T; step 4 is
// then the very same K-major contraction for both directions.
#include "ops_common.cuh"

using namespace kfb;

namespace {
struct TrimulWs {
  __nv_bfloat16 *xn, *ab, *gl, *t;
};
size_t carve(TrimulWs& w, void* base, int batch, int n, int c) {
  Carver cv(base);
  const size_t pos = static_cast<size_t>(batch) * n * n;
  w.xn = cv.take<__nv_bfloat16>(pos * c);  // also reused as tn
  w.ab = cv.take<__nv_bfloat16>(pos * 2 * c);
  w.gl = cv.take<__nv_bfloat16>(pos * c);
  w.t = cv.take<__nv_bfloat16>(pos * c);
  return cv.off;
}
}  // namespace

extern "C" {

KFB_API size_t kfb_trimul_workspace_bytes(int batch, int n, int c) {
  TrimulWs w;
  return carve(w, nullptr, batch, n, c);
}

KFB_API int kfb_trimul_fwd(int incoming, const void* x, const unsigned char* mask, const float* ln_in_w, const float* ln_in_b,
                           const void* w_in_packed, const void* w_gout, const float* ln_out_w, const float* ln_out_b,
                           const void* w_pout, void* out, const void* resid, void* workspace, size_t workspace_bytes,
                           int batch, int n, int c, float eps, int dtype, void* stream_) {
  KFB_CHECK_ARG(x && mask && w_in_packed && w_gout && w_pout && out && workspace, "trimul: null pointer");
  KFB_CHECK_ARG(is_dtype(dtype), "trimul: bad dtype %d", dtype);
  KFB_CHECK_ARG(batch >= 1 && n >= 8 && n % 8 == 0, "trimul: N=%d must be a positive multiple of 8 (pad in the caller)", n);
  KFB_CHECK_ARG(c % 64 == 0 && c >= 64 && c <= 512, "trimul: C=%d must be a multiple of 64 in [64, 512]", c);
  TrimulWs w;
  const size_t need = carve(w, workspace, batch, n, c);
  KFB_CHECK_ARG(workspace_bytes >= need, "trimul: workspace %zu < %zu bytes", workspace_bytes, need);
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "trimul: workspace must be 256-byte aligned");
  cudaStream_t stream = as_stream(stream_);
  const long long nn = static_cast<long long>(n) * n;
  const long long pos = nn * batch;

  // 1. LayerNorm_in
  KFB_TRY(launch_layernorm(stream, x, w.xn, ln_in_w, ln_in_b, pos, c, c, c, eps, dtype, KFB_BF16));

  // 2. input projection, gated, masked, channel-major.  ab[ch][b][o][n]
  {
    GemmParams p = {};
    p.n_extent = n;
    p.o_extent = n;
    p.batch = batch;
    p.n_cols = 4 * c;
    p.k_extent = c;
    p.glu = GLU_SIGMOID;
    p.nseg = 1;
    EpiSeg& s = p.seg[0];
    s.col_begin = 0;
    s.ncols = 2 * c;
    s.out_fp32 = 0;
    s.vec = 0;
    s.dst = w.ab;
    s.s_col = pos;
    s.s_n = 1;
    s.s_o = n;
    s.s_b = nn;
    p.rowmask = mask;
    p.mask_segs = 1;
    p.m_b = nn;
    p.m_o = incoming ? 1 : n;
    p.m_n = incoming ? n : 1;
    GemmOperandA a = {w.xn, incoming ? static_cast<long long>(n) * c : c, incoming ? c : static_cast<long long>(n) * c,
                      nn * c};
    GemmOperandB b = {w_in_packed, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 256, "trimul_in_proj"));
  }
  // 3. output gate logits (natural order)
  {
    GemmParams p = {};
    p.n_extent = static_cast<int>(pos);
    p.o_extent = 1;
    p.batch = 1;
    p.n_cols = c;
    p.k_extent = c;
    p.nseg = 1;
    p.seg[0] = row_major_seg(w.gl, c, c, 0, 0, 0);
    GemmOperandA a = {w.xn, c, 0, 0};
    GemmOperandB b = {w_gout, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "trimul_gate_proj"));
  }
  // 4. contraction: t[ch*B+b][i][j] = sum_k A[i][k] B[j][k]
  {
    GemmParams p = {};
    p.n_extent = n;
    p.o_extent = 1;
    p.batch = c * batch;
    p.n_cols = n;
    p.k_extent = n;
    p.b_batched = 1;
    p.nseg = 1;
    p.seg[0] = row_major_seg(w.t, n, n, 0, nn, 0);
    GemmOperandA a = {w.ab, n, 0, nn};
    GemmOperandB b = {w.ab + static_cast<long long>(c) * pos, n, nn};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "trimul_contraction"));
  }
  // 5. LayerNorm_out: channel-major t -> position-major tn (reuses xn's storage)
  __nv_bfloat16* tn = w.xn;
  KFB_TRY(launch_layernorm_cm(stream, w.t, tn, ln_out_w, ln_out_b, batch, nn, c, pos, nn, eps, KFB_BF16));
  // 6. output projection with sigmoid gate (and optional residual)
  {
    GemmParams p = {};
    p.n_extent = static_cast<int>(pos);
    p.o_extent = 1;
    p.batch = 1;
    p.n_cols = c;
    p.k_extent = c;
    p.nseg = 1;
    p.seg[0] = row_major_seg(out, c, c, 0, 0, dtype == KFB_FP32);
    p.gate = w.gl;
    p.g_col = 1;
    p.g_n = c;
    p.resid = resid;
    GemmOperandA a = {tn, c, 0, 0};
    GemmOperandB b = {w_pout, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "trimul_out_proj"));
  }
  return KFB_OK;
}

}  // extern "C"
