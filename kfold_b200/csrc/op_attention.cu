// Triangle attention (starting / ending node) and pair-bias self-attention as kernel sequences.
//
// Triangle attention:
//   1. LayerNorm                         x -> xn (bf16)
//   2. one projection GEMM of xn with [Wq/sqrt(D) | Wk | Wg | Wv | Wz]:
//        q, k, g      position-major                       (row-major segment)
//        v            transposed per pair row, V^T[h*D+d][k] (channel-major segment) so that it is the
//                     K-major B operand of the P V product
//        triangle bias channel-major [h][j][k]               (channel-major segment)
//   3. flash attention with the bias tile streamed through shared memory, output gated by sigmoid(g)
//   4. output projection GEMM (+ optional residual)
// The ending node is the starting node on the transposed pair tensor: step 2 walks xn with its two
// position strides swapped (a tensor-map change, no data movement), the key mask is read transposed,
// and step 4 scatters its rows back to the untransposed positions.
#include "attention.cuh"
#include "ops_common.cuh"

using namespace kfb;

namespace {

inline int dpad_of(int d) { return d <= 32 ? 32 : 64; }

struct TriattWs {
  __nv_bfloat16 *xn, *qkg, *vt, *bias, *og;
};
size_t carve_triatt(TriattWs& w, void* base, int batch, int n, int c, int heads) {
  Carver cv(base);
  const size_t pos = static_cast<size_t>(batch) * n * n;
  const int hdp = heads * dpad_of(c / heads);
  w.xn = cv.take<__nv_bfloat16>(pos * c);
  w.qkg = cv.take<__nv_bfloat16>(pos * 3 * hdp);
  w.vt = cv.take<__nv_bfloat16>(pos * hdp);
  w.bias = cv.take<__nv_bfloat16>(pos * heads);
  w.og = cv.take<__nv_bfloat16>(pos * c);
  return cv.off;
}

struct ApbWs {
  __nv_bfloat16 *qkg, *vt, *og;
};
size_t carve_apb(ApbWs& w, void* base, int batch, int l, int c, int heads) {
  Carver cv(base);
  const size_t rows = static_cast<size_t>(batch) * l;
  const int hdp = heads * dpad_of(c / heads);
  w.qkg = cv.take<__nv_bfloat16>(rows * 3 * hdp);
  w.vt = cv.take<__nv_bfloat16>(rows * hdp);
  w.og = cv.take<__nv_bfloat16>(rows * c);
  return cv.off;
}

// cross attention (queries and keys from different tensors): [q | g] of the query rows, k and v^T of the key rows
struct ApbCrossWs {
  __nv_bfloat16 *qg, *kk, *vt, *og;
};
size_t carve_apb_cross(ApbCrossWs& w, void* base, int batch, int lq, int lk, int c, int heads) {
  Carver cv(base);
  const size_t rows_q = static_cast<size_t>(batch) * lq, rows_k = static_cast<size_t>(batch) * lk;
  const int hdp = heads * dpad_of(c / heads);
  w.qg = cv.take<__nv_bfloat16>(rows_q * 2 * hdp);
  w.kk = cv.take<__nv_bfloat16>(rows_k * hdp);
  w.vt = cv.take<__nv_bfloat16>(rows_k * hdp);
  w.og = cv.take<__nv_bfloat16>(rows_q * c);
  return cv.off;
}
struct ApbCrossWsPrecise {
  __nv_bfloat16 *xq6, *xk6, *og6;
  float *qg, *kv;
};
size_t carve_apb_cross_precise(ApbCrossWsPrecise& w, void* base, int batch, int lq, int lk, int c) {
  Carver cv(base);
  const size_t rows_q = static_cast<size_t>(batch) * lq, rows_k = static_cast<size_t>(batch) * lk;
  w.xq6 = cv.take<__nv_bfloat16>(rows_q * 6 * c);
  w.xk6 = cv.take<__nv_bfloat16>(rows_k * 6 * c);
  w.og6 = cv.take<__nv_bfloat16>(rows_q * 6 * c);
  w.qg = cv.take<float>(rows_q * 2 * c);
  w.kv = cv.take<float>(rows_k * 2 * c);
  return cv.off;
}

// ------------------------------------------------------------------------------------------------
// fp32-accurate variants (KFB_FP32_PRECISE): split-operand GEMMs around the fp32 attention kernel.
// ------------------------------------------------------------------------------------------------
struct TriattWsPrecise {
  __nv_bfloat16 *xn6, *og6;
  float *qkgv, *bias;
};
size_t carve_triatt_precise(TriattWsPrecise& w, void* base, int batch, int n, int c, int heads) {
  Carver cv(base);
  const size_t pos = static_cast<size_t>(batch) * n * n;
  w.xn6 = cv.take<__nv_bfloat16>(pos * 6 * c);
  w.og6 = cv.take<__nv_bfloat16>(pos * 6 * c);
  w.qkgv = cv.take<float>(pos * 4 * c);
  w.bias = cv.take<float>(pos * heads);
  return cv.off;
}

int triatt_precise(cudaStream_t stream, int ending, const void* x, const unsigned char* mask, const float* ln_w,
                   const float* ln_b, const void* w_proj6, const void* w_out6, void* out, const void* resid,
                   const TriattWsPrecise& w, int batch, int n, int c, int heads, float eps) {
  const int d = c / heads;
  const long long nn = static_cast<long long>(n) * n;
  const long long pos = nn * batch;
  KFB_TRY(launch_layernorm_split(stream, static_cast<const float*>(x), w.xn6, ln_w, ln_b, pos, c, c, eps, 1));
  {
    GemmParams p = {};
    p.n_extent = n;
    p.o_extent = n;
    p.batch = batch;
    p.n_cols = 4 * c + 32;
    p.k_extent = 6 * c;
    p.precise = 1;
    p.nseg = 2;
    p.seg[0] = row_major_seg(w.qkgv, 4 * c, 4 * c, static_cast<long long>(n) * 4 * c, nn * 4 * c, 1, 0);
    EpiSeg& sb = p.seg[1];
    sb = {};
    sb.col_begin = 4 * c;
    sb.ncols = heads;
    sb.out_fp32 = 1;
    sb.dst = w.bias;
    sb.s_col = nn;
    sb.s_n = 1;
    sb.s_o = n;
    sb.s_b = static_cast<long long>(heads) * nn;
    const long long c6 = 6ll * c;
    GemmOperandA a = {w.xn6, ending ? n * c6 : c6, ending ? c6 : n * c6, nn * c6};
    GemmOperandB b = {w_proj6, c6, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 128, "triatt_proj_precise"));
  }
  {
    AttnFp32Params p = {};
    p.batch = batch * n;
    p.heads = heads;
    p.lq = n;
    p.lk = n;
    p.d = d;
    p.q = p.k = p.v = p.g = w.qkgv;
    p.ld = 4 * c;
    p.q_col0 = 0; p.k_col0 = c; p.g_col0 = 2 * c; p.v_col0 = 3 * c;
    p.bias = w.bias; p.ldb = n; p.bias_div = n;
    p.mask = mask;
    p.mask_lo_extent = n;
    p.m_hi = nn;
    p.m_lo = ending ? 1 : n;
    p.m_k = ending ? n : 1;
    p.out6 = w.og6;
    p.tag = "triatt_attention_fp32";
    KFB_TRY(launch_attention_fp32(stream, p));
  }
  {
    GemmParams p = {};
    p.n_extent = n;
    p.o_extent = n;
    p.batch = batch;
    p.n_cols = c;
    p.k_extent = 6 * c;
    p.precise = 1;
    p.nseg = 1;
    p.seg[0] = row_major_seg(out, c, ending ? static_cast<long long>(n) * c : c, ending ? c : static_cast<long long>(n) * c,
                             nn * c, 1);
    p.resid = resid;
    const long long c6 = 6ll * c;
    GemmOperandA a = {w.og6, c6, n * c6, nn * c6};
    GemmOperandB b = {w_out6, c6, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "triatt_out_proj_precise"));
  }
  return KFB_OK;
}

struct ApbWsPrecise {
  __nv_bfloat16 *x6, *og6;
  float* qkgv;
};
size_t carve_apb_precise(ApbWsPrecise& w, void* base, int batch, int l, int c) {
  Carver cv(base);
  const size_t rows = static_cast<size_t>(batch) * l;
  w.x6 = cv.take<__nv_bfloat16>(rows * 6 * c);
  w.og6 = cv.take<__nv_bfloat16>(rows * 6 * c);
  w.qkgv = cv.take<float>(rows * 4 * c);
  return cv.off;
}

}  // namespace

extern "C" {

KFB_API size_t kfb_triatt_workspace_bytes_precise(int batch, int n, int c, int heads) {
  TriattWsPrecise w;
  return carve_triatt_precise(w, nullptr, batch, n, c, heads);
}

KFB_API size_t kfb_apb_workspace_bytes_precise(int batch, int l, int c) {
  ApbWsPrecise w;
  return carve_apb_precise(w, nullptr, batch, l, c);
}

KFB_API size_t kfb_pair_bias_workspace_bytes_precise(int batch, int n, int c) {
  return align_up(static_cast<size_t>(batch) * n * n * 6 * c * sizeof(__nv_bfloat16), 256);
}

KFB_API size_t kfb_triatt_workspace_bytes(int batch, int n, int c, int heads) {
  TriattWs w;
  return carve_triatt(w, nullptr, batch, n, c, heads);
}

KFB_API int kfb_triatt_fwd(int ending, const void* x, const unsigned char* mask, const float* ln_w, const float* ln_b,
                           const void* w_proj_packed, const void* w_out, void* out, const void* resid, void* workspace,
                           size_t workspace_bytes, int batch, int n, int c, int heads, float eps, int dtype, void* stream_) {
  KFB_CHECK_ARG(x && mask && w_proj_packed && w_out && out && workspace, "triatt: null pointer");
  KFB_CHECK_ARG(is_dtype(dtype), "triatt: bad dtype %d", dtype);
  KFB_CHECK_ARG(batch >= 1 && n >= 8 && n % 8 == 0, "triatt: N=%d must be a positive multiple of 8 (pad in the caller)", n);
  KFB_CHECK_ARG(heads >= 1 && c % heads == 0 && c % 8 == 0, "triatt: C=%d heads=%d", c, heads);
  const int d = c / heads;
  KFB_CHECK_ARG(d % 8 == 0 && d >= 16 && d <= 64, "triatt: head dim %d not in {16, 24, ..., 64}", d);
  KFB_CHECK_ARG(static_cast<long long>(batch) * n <= 65535, "triatt: batch*N = %lld exceeds 65535", static_cast<long long>(batch) * n);
  if (dtype == KFB_FP32_PRECISE) {
    TriattWsPrecise wp;
    const size_t need_p = carve_triatt_precise(wp, workspace, batch, n, c, heads);
    KFB_CHECK_ARG(workspace_bytes >= need_p, "triatt: workspace %zu < %zu bytes", workspace_bytes, need_p);
    KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "triatt: workspace must be 256-byte aligned");
    return triatt_precise(as_stream(stream_), ending, x, mask, ln_w, ln_b, w_proj_packed, w_out, out, resid, wp, batch, n, c,
                          heads, eps);
  }
  const int dp = dpad_of(d), hdp = heads * dp;
  TriattWs w;
  const size_t need = carve_triatt(w, workspace, batch, n, c, heads);
  KFB_CHECK_ARG(workspace_bytes >= need, "triatt: workspace %zu < %zu bytes", workspace_bytes, need);
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "triatt: workspace must be 256-byte aligned");
  cudaStream_t stream = as_stream(stream_);
  const long long nn = static_cast<long long>(n) * n;
  const long long pos = nn * batch;

  KFB_TRY(launch_layernorm(stream, x, w.xn, ln_w, ln_b, pos, c, c, c, eps, dtype, KFB_BF16));
  // projection: rows walked as (b, o, n); for the ending node (o, n) = (second, first) pair index
  {
    GemmParams p = {};
    p.n_extent = n;
    p.o_extent = n;
    p.batch = batch;
    p.n_cols = 4 * hdp + 32;
    p.k_extent = c;
    p.nseg = 3;
    p.seg[0] = row_major_seg(w.qkg, 3 * hdp, 3 * hdp, static_cast<long long>(n) * 3 * hdp, nn * 3 * hdp, 0, 0);
    EpiSeg& sv = p.seg[1];
    sv = {};
    sv.col_begin = 3 * hdp;
    sv.ncols = hdp;
    sv.dst = w.vt;
    sv.s_col = n;
    sv.s_n = 1;
    sv.s_o = static_cast<long long>(hdp) * n;
    sv.s_b = static_cast<long long>(hdp) * nn;
    EpiSeg& sb = p.seg[2];
    sb = {};
    sb.col_begin = 4 * hdp;
    sb.ncols = heads;
    sb.dst = w.bias;
    sb.s_col = nn;
    sb.s_n = 1;
    sb.s_o = n;
    sb.s_b = static_cast<long long>(heads) * nn;
    GemmOperandA a = {w.xn, ending ? static_cast<long long>(n) * c : c, ending ? c : static_cast<long long>(n) * c, nn * c};
    GemmOperandB b = {w_proj_packed, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 128, "triatt_proj"));
  }
  {
    AttnParams p = {};
    p.batch = batch * n;
    p.heads = heads;
    p.lq = n;
    p.lk = n;
    p.d = d;
    p.dpad = dp;
    p.q = w.qkg; p.ldq = 3 * hdp; p.q_col0 = 0;
    p.k = w.qkg; p.ldk = 3 * hdp; p.k_col0 = hdp;
    p.g = w.qkg; p.ldg = 3 * hdp; p.g_col0 = 2 * hdp;
    p.vt = w.vt; p.ldv = n;
    p.bias = w.bias; p.ldb = n; p.bias_div = n;
    p.mask = mask;
    p.mask_lo_extent = n;
    p.m_hi = nn;
    p.m_lo = ending ? 1 : n;
    p.m_k = ending ? n : 1;
    p.out = w.og; p.ldo = c;
    p.tag = "triatt_attention";
    KFB_TRY(launch_attention(stream, p));
  }
  {
    GemmParams p = {};
    p.n_extent = n;
    p.o_extent = n;
    p.batch = batch;
    p.n_cols = c;
    p.k_extent = c;
    p.nseg = 1;
    // row (b, o, n) goes back to pair position (o, n) for the starting node, (n, o) for the ending node
    p.seg[0] = row_major_seg(out, c, ending ? static_cast<long long>(n) * c : c, ending ? c : static_cast<long long>(n) * c,
                             nn * c, dtype == KFB_FP32);
    p.resid = resid;
    GemmOperandA a = {w.og, c, static_cast<long long>(n) * c, nn * c};
    GemmOperandB b = {w_out, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "triatt_out_proj"));
  }
  return KFB_OK;
}

// ------------------------------------------------------------------------------------------------
// Row-sharded triangle attention (starting-node form on a shard of `rows` of the n pair rows; the ending
// node is the same on the transposed shard).  "project" is local; the triangle bias it produces covers only
// the shard's rows [h][rows][n] and the caller all-gathers it per head into [h][n][n]; "finish" runs the
// attention of the local rows against the full bias and projects the result.
// ------------------------------------------------------------------------------------------------
KFB_API int kfb_triatt_project(const void* x, const float* ln_w, const float* ln_b, const void* w_proj_packed,
                               void* xn_scratch, void* qkg_out, void* vt_out, void* bias_out, int rows, int n, int c,
                               int heads, int exchange_layout, float eps, int dtype, void* stream_) {
  KFB_CHECK_ARG(x && w_proj_packed && (xn_scratch || exchange_layout) && qkg_out && vt_out && bias_out, "triatt_project: null pointer");
  KFB_CHECK_ARG(!exchange_layout || n % rows == 0, "triatt_project: the exchange layout needs N=%d to be a multiple of rows=%d", n, rows);
  KFB_CHECK_ARG(is_dtype(dtype), "triatt_project: bad dtype %d", dtype);
  KFB_CHECK_ARG(rows >= 1 && rows <= n && n >= 8 && n % 8 == 0, "triatt_project: rows=%d N=%d", rows, n);
  KFB_CHECK_ARG(heads >= 1 && c % heads == 0 && c % 8 == 0, "triatt_project: C=%d heads=%d", c, heads);
  const int d = c / heads;
  KFB_CHECK_ARG(d % 8 == 0 && d >= 16 && d <= 64, "triatt_project: head dim %d not in {16, 24, ..., 64}", d);
  const int dp = dpad_of(d), hdp = heads * dp;
  cudaStream_t stream = as_stream(stream_);
  const long long rn = static_cast<long long>(rows) * n;
  __nv_bfloat16* xn = static_cast<__nv_bfloat16*>(xn_scratch);
  if (exchange_layout) {
    // x: the normalised rows as an all-to-all of kfb_layernorm_exchange's output leaves them, [q][i_q][j][c] holding row j of
    // this (transposed) shard at position q * rows + i_q.  GEMM row = (batch j, o q, n i_q); outputs in the usual order.
    GemmParams p = {};
    p.n_extent = rows;
    p.o_extent = n / rows;
    p.batch = rows;
    p.n_cols = 4 * hdp + 32;
    p.k_extent = c;
    p.nseg = 3;
    p.seg[0] = row_major_seg(qkg_out, 3 * hdp, 3 * hdp, static_cast<long long>(rows) * 3 * hdp, static_cast<long long>(n) * 3 * hdp, 0, 0);
    EpiSeg& sv = p.seg[1];
    sv = {};
    sv.col_begin = 3 * hdp;
    sv.ncols = hdp;
    sv.dst = vt_out;
    sv.s_col = n;
    sv.s_n = 1;
    sv.s_o = rows;
    sv.s_b = static_cast<long long>(hdp) * n;
    EpiSeg& sb = p.seg[2];
    sb = {};
    sb.col_begin = 4 * hdp;
    sb.ncols = heads;
    sb.dst = bias_out;
    sb.s_col = rn;
    sb.s_n = 1;
    sb.s_o = rows;
    sb.s_b = n;
    GemmOperandA a = {x, static_cast<long long>(rows) * c, static_cast<long long>(rows) * rows * c, c};
    GemmOperandB b = {w_proj_packed, c, 0};
    return launch_gemm_bf16(stream, a, b, p, 128, "triatt_proj");
  }
  KFB_TRY(launch_layernorm(stream, x, xn, ln_w, ln_b, rn, c, c, c, eps, dtype, KFB_BF16));
  GemmParams p = {};
  p.n_extent = n;
  p.o_extent = rows;
  p.batch = 1;
  p.n_cols = 4 * hdp + 32;
  p.k_extent = c;
  p.nseg = 3;
  p.seg[0] = row_major_seg(qkg_out, 3 * hdp, 3 * hdp, static_cast<long long>(n) * 3 * hdp, 0, 0, 0);
  EpiSeg& sv = p.seg[1];
  sv = {};
  sv.col_begin = 3 * hdp;
  sv.ncols = hdp;
  sv.dst = vt_out;
  sv.s_col = n;
  sv.s_n = 1;
  sv.s_o = static_cast<long long>(hdp) * n;
  EpiSeg& sb = p.seg[2];
  sb = {};
  sb.col_begin = 4 * hdp;
  sb.ncols = heads;
  sb.dst = bias_out;
  sb.s_col = rn;
  sb.s_n = 1;
  sb.s_o = n;
  GemmOperandA a = {xn, c, static_cast<long long>(n) * c, 0};
  GemmOperandB b = {w_proj_packed, c, 0};
  return launch_gemm_bf16(stream, a, b, p, 128, "triatt_proj");
}

KFB_API int kfb_triatt_finish(const void* qkg, const void* vt, const void* bias_full, const unsigned char* mask,
                              const void* w_out, void* og_scratch, void* out, const void* resid, int rows, int n, int c,
                              int heads, int exchange_layout, int dtype, void* stream_) {
  KFB_CHECK_ARG(!exchange_layout || (n % rows == 0 && resid == nullptr && dtype == KFB_BF16),
                "triatt_finish: the exchange layout takes N=%d a multiple of rows=%d, bf16, no residual", n, rows);
  KFB_CHECK_ARG(qkg && vt && bias_full && mask && w_out && og_scratch && out, "triatt_finish: null pointer");
  KFB_CHECK_ARG(is_dtype(dtype), "triatt_finish: bad dtype %d", dtype);
  KFB_CHECK_ARG(rows >= 1 && rows <= n && rows <= 65535 && n >= 8 && n % 8 == 0, "triatt_finish: rows=%d N=%d", rows, n);
  const int d = c / heads;
  const int dp = dpad_of(d), hdp = heads * dp;
  cudaStream_t stream = as_stream(stream_);
  {
    AttnParams p = {};
    p.batch = rows;
    p.heads = heads;
    p.lq = n;
    p.lk = n;
    p.d = d;
    p.dpad = dp;
    p.q = qkg; p.ldq = 3 * hdp; p.q_col0 = 0;
    p.k = qkg; p.ldk = 3 * hdp; p.k_col0 = hdp;
    p.g = qkg; p.ldg = 3 * hdp; p.g_col0 = 2 * hdp;
    p.vt = vt; p.ldv = n;
    p.bias = bias_full; p.ldb = n; p.bias_div = rows;
    p.mask = mask;
    p.mask_lo_extent = rows;
    p.m_hi = 0;
    p.m_lo = n;
    p.m_k = 1;
    p.out = og_scratch; p.ldo = c;
    p.tag = "triatt_attention";
    KFB_TRY(launch_attention(stream, p));
  }
  GemmParams p = {};
  p.n_extent = static_cast<int>(static_cast<long long>(rows) * n);
  p.o_extent = 1;
  p.batch = 1;
  p.n_cols = c;
  p.k_extent = c;
  p.nseg = 1;
  p.seg[0] = row_major_seg(out, c, c, 0, 0, dtype == KFB_FP32);
  p.resid = resid;
  GemmOperandA a = {og_scratch, c, 0, 0};
  GemmOperandB b = {w_out, c, 0};
  if (exchange_layout) {
    // out[q][j][k_q][c] = update of position (j, q * rows + k_q): the send buffer of the transpose back, block q for rank q
    p.n_extent = rows;
    p.o_extent = n / rows;
    p.batch = rows;
    p.seg[0] = row_major_seg(out, c, c, static_cast<long long>(rows) * rows * c, static_cast<long long>(rows) * c, 0);
    a = {og_scratch, c, static_cast<long long>(rows) * c, static_cast<long long>(n) * c};
  }
  return launch_gemm_bf16(stream, a, b, p, 0, "triatt_out_proj");
}

KFB_API size_t kfb_pair_bias_workspace_bytes(int batch, int n, int c) {
  return align_up(static_cast<size_t>(batch) * n * n * c * sizeof(__nv_bfloat16), 256);
}

// bias[b][h][i][j] = sum_c LN(z)[b][i][j][c] * W[h][c], stored bf16 head-major; with `transposed` the
// last two indices are swapped (bias_out[b][h][j][i]).  z is (batch, rows, n, c): square on one GPU,
// a row shard (rows < n) otherwise.
static int pair_bias_impl(const void* z, const float* ln_w, const float* ln_b, const void* w, void* bias_out,
                          void* workspace, int batch, int rows, int n, int c, int heads, int transposed, float eps,
                          int dtype, cudaStream_t stream) {
  const long long rn = static_cast<long long>(rows) * n;
  __nv_bfloat16* zn = static_cast<__nv_bfloat16*>(workspace);
  KFB_TRY(launch_layernorm(stream, z, zn, ln_w, ln_b, rn * batch, c, c, c, eps, dtype, KFB_BF16));
  GemmParams p = {};
  p.n_extent = n;
  p.o_extent = rows;
  p.batch = batch;
  p.n_cols = heads;
  p.k_extent = c;
  p.nseg = 1;
  EpiSeg& s = p.seg[0];
  s.col_begin = 0;
  s.ncols = heads;
  s.dst = bias_out;
  s.s_col = rn;
  s.s_n = transposed ? rows : 1;
  s.s_o = transposed ? 1 : n;
  s.s_b = static_cast<long long>(heads) * rn;
  GemmOperandA a = {zn, c, static_cast<long long>(n) * c, rn * c};
  GemmOperandB b = {w, c, 0};
  return launch_gemm_bf16(stream, a, b, p, 0, "pair_bias_proj");
}

KFB_API int kfb_pair_bias_fwd(const void* z, const float* ln_w, const float* ln_b, const void* w, void* bias_out,
                              void* workspace, size_t workspace_bytes, int batch, int n, int c, int heads, int transposed,
                              float eps, int dtype, void* stream_) {
  KFB_CHECK_ARG(z && w && bias_out && workspace, "pair_bias: null pointer");
  KFB_CHECK_ARG(is_dtype(dtype), "pair_bias: bad dtype %d", dtype);
  KFB_CHECK_ARG(batch >= 1 && n >= 8 && n % 8 == 0 && c % 8 == 0 && heads >= 1, "pair_bias: batch %d n %d c %d heads %d",
                batch, n, c, heads);
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "pair_bias: workspace must be 256-byte aligned");
  if (dtype == KFB_FP32_PRECISE) {
    // fp32 in, fp32 bias out, split-operand GEMM
    KFB_CHECK_ARG(workspace_bytes >= kfb_pair_bias_workspace_bytes_precise(batch, n, c), "pair_bias: workspace too small");
    cudaStream_t stream = as_stream(stream_);
    const long long nn = static_cast<long long>(n) * n;
    __nv_bfloat16* zn6 = static_cast<__nv_bfloat16*>(workspace);
    KFB_TRY(launch_layernorm_split(stream, static_cast<const float*>(z), zn6, ln_w, ln_b, nn * batch, c, c, eps, 1));
    GemmParams p = {};
    p.n_extent = n;
    p.o_extent = n;
    p.batch = batch;
    p.n_cols = heads;
    p.k_extent = 6 * c;
    p.precise = 1;
    p.nseg = 1;
    EpiSeg& sg = p.seg[0];
    sg.col_begin = 0;
    sg.ncols = heads;
    sg.out_fp32 = 1;
    sg.dst = bias_out;
    sg.s_col = nn;
    sg.s_n = transposed ? n : 1;
    sg.s_o = transposed ? 1 : n;
    sg.s_b = static_cast<long long>(heads) * nn;
    const long long c6 = 6ll * c;
    GemmOperandA a = {zn6, c6, n * c6, nn * c6};
    GemmOperandB b = {w, c6, 0};
    return launch_gemm_bf16(stream, a, b, p, 0, "pair_bias_proj_precise");
  }
  KFB_CHECK_ARG(workspace_bytes >= kfb_pair_bias_workspace_bytes(batch, n, c), "pair_bias: workspace too small");
  return pair_bias_impl(z, ln_w, ln_b, w, bias_out, workspace, batch, n, n, c, heads, transposed, eps, dtype, as_stream(stream_));
}

// Row-shard form: z (rows, n, c) -> bias_out bf16 [heads][rows][n].  workspace: rows*n*c bf16.
KFB_API int kfb_pair_bias_rows_fwd(const void* z, const float* ln_w, const float* ln_b, const void* w, void* bias_out,
                                   void* workspace, size_t workspace_bytes, int rows, int n, int c, int heads, float eps,
                                   int dtype, void* stream_) {
  KFB_CHECK_ARG(z && w && bias_out && workspace, "pair_bias_rows: null pointer");
  KFB_CHECK_ARG(is_dtype(dtype), "pair_bias_rows: bad dtype %d", dtype);
  KFB_CHECK_ARG(rows >= 1 && rows <= n && n >= 8 && n % 8 == 0 && c % 8 == 0 && heads >= 1,
                "pair_bias_rows: rows %d n %d c %d heads %d", rows, n, c, heads);
  KFB_CHECK_ARG(workspace_bytes >= static_cast<size_t>(rows) * n * c * sizeof(__nv_bfloat16), "pair_bias_rows: workspace too small");
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "pair_bias_rows: workspace must be 256-byte aligned");
  return pair_bias_impl(z, ln_w, ln_b, w, bias_out, workspace, 1, rows, n, c, heads, 0, eps, dtype, as_stream(stream_));
}

KFB_API size_t kfb_apb_workspace_bytes(int batch, int l, int c, int heads) {
  ApbWs w;
  return carve_apb(w, nullptr, batch, l, c, heads);
}

KFB_API int kfb_apb_fwd(const void* x, const void* pair_bias, const unsigned char* mask, const void* w_proj_packed,
                        const float* proj_bias, const void* w_out, const float* out_bias, const void* out_gate,
                        int gate_share, long long gate_ld, void* out, const void* resid, void* workspace,
                        size_t workspace_bytes, int batch, int l, int c, int heads, int bias_div, int out_dtype, void* stream_) {
  KFB_CHECK_ARG(x && pair_bias && mask && w_proj_packed && w_out && out && workspace, "apb: null pointer");
  KFB_CHECK_ARG(is_dtype(out_dtype), "apb: bad dtype %d", out_dtype);
  KFB_CHECK_ARG(batch >= 1 && l >= 8 && l % 8 == 0, "apb: L=%d must be a positive multiple of 8 (pad in the caller)", l);
  KFB_CHECK_ARG(heads >= 1 && c % heads == 0 && c % 8 == 0, "apb: c=%d heads=%d", c, heads);
  KFB_CHECK_ARG(bias_div >= 1 && batch % bias_div == 0, "apb: batch %d not a multiple of bias_div %d", batch, bias_div);
  if (out_gate != nullptr)
    KFB_CHECK_ARG(gate_share >= 1 && batch % gate_share == 0, "apb: batch %d not a multiple of gate_share %d", batch, gate_share);
  else
    gate_share = 1;
  if (gate_ld <= 0) gate_ld = c;
  KFB_CHECK_ARG(gate_ld >= c, "apb: gate row stride %lld below c=%d", gate_ld, c);
  KFB_CHECK_ARG(out_gate == nullptr || out_dtype == KFB_FP32_PRECISE || (gate_ld % 8 == 0 && (reinterpret_cast<uintptr_t>(out_gate) & 15) == 0),
                "apb: bf16 gate rows must start on 16-byte boundaries (pointer and row stride %lld)", gate_ld);
  const int d = c / heads;
  KFB_CHECK_ARG(d % 8 == 0 && d >= 16 && d <= 64, "apb: head dim %d not in {16, 24, ..., 64}", d);
  if (out_dtype == KFB_FP32_PRECISE) {
    // everything fp32: x, pair_bias, out_gate logits, out, resid; weights from the precise packing
    ApbWsPrecise wp;
    const size_t need_p = carve_apb_precise(wp, workspace, batch, l, c);
    KFB_CHECK_ARG(workspace_bytes >= need_p, "apb: workspace %zu < %zu bytes", workspace_bytes, need_p);
    KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "apb: workspace must be 256-byte aligned");
    cudaStream_t stream = as_stream(stream_);
    const long long rows = static_cast<long long>(batch) * l;
    const long long c6 = 6ll * c;
    KFB_TRY(launch_layernorm_split(stream, static_cast<const float*>(x), wp.x6, nullptr, nullptr, rows, c, c, 0.f, 0));
    {
      GemmParams p = {};
      p.n_extent = static_cast<int>(rows);
      p.o_extent = 1;
      p.batch = 1;
      p.n_cols = 4 * c;
      p.k_extent = 6 * c;
      p.precise = 1;
      p.nseg = 1;
      p.seg[0] = row_major_seg(wp.qkgv, 4 * c, 4 * c, 0, 0, 1);
      p.col_bias = proj_bias;
      GemmOperandA a = {wp.x6, c6, 0, 0};
      GemmOperandB b = {w_proj_packed, c6, 0};
      KFB_TRY(launch_gemm_bf16(stream, a, b, p, 128, "apb_proj_precise"));
    }
    {
      AttnFp32Params p = {};
      p.batch = batch;
      p.heads = heads;
      p.lq = l;
      p.lk = l;
      p.d = d;
      p.q = p.k = p.v = p.g = wp.qkgv;
      p.ld = 4 * c;
      p.q_col0 = 0; p.k_col0 = c; p.g_col0 = 2 * c; p.v_col0 = 3 * c;
      p.bias = static_cast<const float*>(pair_bias); p.ldb = l; p.bias_div = bias_div;
      p.mask = mask;
      p.mask_lo_extent = 1;
      p.m_hi = l;
      p.m_lo = 0;
      p.m_k = 1;
      p.out6 = wp.og6;
      p.tag = "apb_attention_fp32";
      KFB_TRY(launch_attention_fp32(stream, p));
    }
    GemmParams p = {};
    p.n_extent = l;
    p.o_extent = gate_share;
    p.batch = batch / gate_share;
    p.n_cols = c;
    p.k_extent = 6 * c;
    p.precise = 1;
    p.nseg = 1;
    const long long lc = static_cast<long long>(l) * c;
    p.seg[0] = row_major_seg(out, c, c, lc, lc * gate_share, 1);
    p.col_bias = out_bias;
    p.resid = resid;
    if (out_gate != nullptr) {
      p.gate = static_cast<const __nv_bfloat16*>(out_gate);  // fp32 logits in this mode
      p.g_col = 1;
      p.g_n = gate_ld;
      p.g_o = 0;
      p.g_b = l * gate_ld;
    }
    GemmOperandA a = {wp.og6, c6, l * c6, l * c6 * gate_share};
    GemmOperandB b = {w_out, c6, 0};
    return launch_gemm_bf16(stream, a, b, p, 0, "apb_out_proj_precise");
  }
  const int dp = dpad_of(d), hdp = heads * dp;
  ApbWs w;
  const size_t need = carve_apb(w, workspace, batch, l, c, heads);
  KFB_CHECK_ARG(workspace_bytes >= need, "apb: workspace %zu < %zu bytes", workspace_bytes, need);
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "apb: workspace must be 256-byte aligned");
  cudaStream_t stream = as_stream(stream_);
  {
    GemmParams p = {};
    p.n_extent = l;
    p.o_extent = batch;
    p.batch = 1;
    p.n_cols = 4 * hdp;
    p.k_extent = c;
    p.nseg = 2;
    p.seg[0] = row_major_seg(w.qkg, 3 * hdp, 3 * hdp, static_cast<long long>(l) * 3 * hdp, 0, 0, 0);
    EpiSeg& sv = p.seg[1];
    sv = {};
    sv.col_begin = 3 * hdp;
    sv.ncols = hdp;
    sv.dst = w.vt;
    sv.s_col = l;
    sv.s_n = 1;
    sv.s_o = static_cast<long long>(hdp) * l;
    p.col_bias = proj_bias;
    GemmOperandA a = {x, c, static_cast<long long>(l) * c, 0};
    GemmOperandB b = {w_proj_packed, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 128, "apb_proj"));
  }
  {
    AttnParams p = {};
    p.batch = batch;
    p.heads = heads;
    p.lq = l;
    p.lk = l;
    p.d = d;
    p.dpad = dp;
    p.q = w.qkg; p.ldq = 3 * hdp; p.q_col0 = 0;
    p.k = w.qkg; p.ldk = 3 * hdp; p.k_col0 = hdp;
    p.g = w.qkg; p.ldg = 3 * hdp; p.g_col0 = 2 * hdp;
    p.vt = w.vt; p.ldv = l;
    p.bias = pair_bias; p.ldb = l; p.bias_div = bias_div;
    p.mask = mask;
    p.mask_lo_extent = 1;
    p.m_hi = l;
    p.m_lo = 0;
    p.m_k = 1;
    p.out = w.og; p.ldo = c;
    p.tag = "apb_attention";
    KFB_TRY(launch_attention(stream, p));
  }
  {
    // rows walked as (group, member, position): `gate_share` consecutive batch entries share one gate row set
    GemmParams p = {};
    p.n_extent = l;
    p.o_extent = gate_share;
    p.batch = batch / gate_share;
    p.n_cols = c;
    p.k_extent = c;
    p.nseg = 1;
    const long long lc = static_cast<long long>(l) * c;
    p.seg[0] = row_major_seg(out, c, c, lc, lc * gate_share, out_dtype == KFB_FP32);
    p.col_bias = out_bias;
    p.resid = resid;
    if (out_gate != nullptr) {
      p.gate = static_cast<const __nv_bfloat16*>(out_gate);
      p.g_col = 1;
      p.g_n = gate_ld;
      p.g_o = 0;
      p.g_b = l * gate_ld;
    }
    GemmOperandA a = {w.og, c, lc, lc * gate_share};
    GemmOperandB b = {w_out, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "apb_out_proj"));
  }
  return KFB_OK;
}

KFB_API size_t kfb_apb_cross_workspace_bytes(int batch, int lq, int lk, int c, int heads) {
  ApbCrossWs w;
  return carve_apb_cross(w, nullptr, batch, lq, lk, c, heads);
}

KFB_API size_t kfb_apb_cross_workspace_bytes_precise(int batch, int lq, int lk, int c) {
  ApbCrossWsPrecise w;
  return carve_apb_cross_precise(w, nullptr, batch, lq, lk, c);
}

KFB_API int kfb_apb_cross_fwd(const void* x_q, const void* x_k, const void* pair_bias, const unsigned char* mask,
                              const void* w_q_packed, const float* q_bias, const void* w_kv_packed, const void* w_out,
                              const float* out_bias, const void* out_gate, long long gate_rows, long long gate_ld, void* out,
                              const void* resid, void* workspace, size_t workspace_bytes, int batch, int lq, int lk, int c, int heads,
                              int bias_div, int bias_mod, int bias_head_major, int out_dtype, void* stream_) {
  KFB_CHECK_ARG(x_q && x_k && pair_bias && mask && w_q_packed && w_kv_packed && w_out && out && workspace,
                "apb_cross: null pointer");
  KFB_CHECK_ARG(is_dtype(out_dtype), "apb_cross: bad dtype %d", out_dtype);
  KFB_CHECK_ARG(batch >= 1 && lq >= 8 && lq % 8 == 0 && lk >= 8 && lk % 8 == 0,
                "apb_cross: Lq=%d and Lk=%d must be positive multiples of 8 (pad in the caller)", lq, lk);
  KFB_CHECK_ARG(heads >= 1 && c % heads == 0 && c % 8 == 0, "apb_cross: c=%d heads=%d", c, heads);
  KFB_CHECK_ARG(bias_div >= 1 && bias_mod >= 0 && bias_head_major >= 0, "apb_cross: bias_div %d bias_mod %d bias_head_major %d",
                bias_div, bias_mod, bias_head_major);
  const int d = c / heads;
  KFB_CHECK_ARG(d % 8 == 0 && d >= 16 && d <= 64, "apb_cross: head dim %d not in {16, 24, ..., 64}", d);
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "apb_cross: workspace must be 256-byte aligned");
  cudaStream_t stream = as_stream(stream_);
  const long long rows_q = static_cast<long long>(batch) * lq, rows_k = static_cast<long long>(batch) * lk;
  if (out_gate == nullptr || gate_rows <= 0) gate_rows = rows_q;
  if (gate_ld <= 0) gate_ld = c;
  KFB_CHECK_ARG(gate_ld >= c, "apb_cross: gate row stride %lld below c=%d", gate_ld, c);
  KFB_CHECK_ARG(out_gate == nullptr || out_dtype == KFB_FP32_PRECISE || (gate_ld % 8 == 0 && (reinterpret_cast<uintptr_t>(out_gate) & 15) == 0),
                "apb_cross: bf16 gate rows must start on 16-byte boundaries (pointer and row stride %lld)", gate_ld);
  KFB_CHECK_ARG(rows_q % gate_rows == 0 && gate_rows < (1ll << 31), "apb_cross: %lld query rows are not a multiple of gate_rows %lld",
                rows_q, gate_rows);
  const int gate_reps = static_cast<int>(rows_q / gate_rows);
  if (out_dtype == KFB_FP32_PRECISE) {
    ApbCrossWsPrecise wp;
    const size_t need_p = carve_apb_cross_precise(wp, workspace, batch, lq, lk, c);
    KFB_CHECK_ARG(workspace_bytes >= need_p, "apb_cross: workspace %zu < %zu bytes", workspace_bytes, need_p);
    const long long c6 = 6ll * c;
    KFB_TRY(launch_layernorm_split(stream, static_cast<const float*>(x_q), wp.xq6, nullptr, nullptr, rows_q, c, c, 0.f, 0));
    KFB_TRY(launch_layernorm_split(stream, static_cast<const float*>(x_k), wp.xk6, nullptr, nullptr, rows_k, c, c, 0.f, 0));
    for (int side = 0; side < 2; ++side) {
      GemmParams p = {};
      p.n_extent = static_cast<int>(side == 0 ? rows_q : rows_k);
      p.o_extent = 1;
      p.batch = 1;
      p.n_cols = 2 * c;
      p.k_extent = 6 * c;
      p.precise = 1;
      p.nseg = 1;
      p.seg[0] = row_major_seg(side == 0 ? wp.qg : wp.kv, 2 * c, 2 * c, 0, 0, 1);
      p.col_bias = side == 0 ? q_bias : nullptr;
      GemmOperandA a = {side == 0 ? wp.xq6 : wp.xk6, c6, 0, 0};
      GemmOperandB b = {side == 0 ? w_q_packed : w_kv_packed, c6, 0};
      KFB_TRY(launch_gemm_bf16(stream, a, b, p, 128, side == 0 ? "apb_cross_q_proj_precise" : "apb_cross_kv_proj_precise"));
    }
    {
      AttnFp32Params p = {};
      p.batch = batch;
      p.heads = heads;
      p.lq = lq;
      p.lk = lk;
      p.d = d;
      p.q = p.g = wp.qg;
      p.k = p.v = wp.kv;
      p.ld = 2 * c;
      p.ld_kv = 2 * c;
      p.q_col0 = 0; p.g_col0 = c; p.k_col0 = 0; p.v_col0 = c;
      p.bias = static_cast<const float*>(pair_bias); p.ldb = lk; p.bias_div = bias_div; p.bias_mod = bias_mod; p.bias_head_major = bias_head_major;
      p.mask = mask;
      p.mask_lo_extent = 1;
      p.m_hi = lk;
      p.m_lo = 0;
      p.m_k = 1;
      p.out6 = wp.og6;
      p.tag = "apb_cross_attention_fp32";
      KFB_TRY(launch_attention_fp32(stream, p));
    }
    GemmParams p = {};
    p.n_extent = static_cast<int>(gate_rows);
    p.o_extent = gate_reps;
    p.batch = 1;
    p.n_cols = c;
    p.k_extent = 6 * c;
    p.precise = 1;
    p.nseg = 1;
    p.seg[0] = row_major_seg(out, c, c, gate_rows * c, 0, 1);
    p.col_bias = out_bias;
    p.resid = resid;
    if (out_gate != nullptr) {
      p.gate = static_cast<const __nv_bfloat16*>(out_gate);  // fp32 logits in this mode; query row r uses row r % gate_rows
      p.g_col = 1;
      p.g_n = gate_ld;
      p.g_o = 0;
      p.g_b = 0;
    }
    GemmOperandA a = {wp.og6, c6, gate_rows * c6, 0};
    GemmOperandB b = {w_out, c6, 0};
    return launch_gemm_bf16(stream, a, b, p, 0, "apb_cross_out_proj_precise");
  }
  const int dp = dpad_of(d), hdp = heads * dp;
  ApbCrossWs w;
  const size_t need = carve_apb_cross(w, workspace, batch, lq, lk, c, heads);
  KFB_CHECK_ARG(workspace_bytes >= need, "apb_cross: workspace %zu < %zu bytes", workspace_bytes, need);
  {
    // query side: [q * log2(e)/sqrt(d) | gate logits]
    GemmParams p = {};
    p.n_extent = static_cast<int>(rows_q);
    p.o_extent = 1;
    p.batch = 1;
    p.n_cols = 2 * hdp;
    p.k_extent = c;
    p.nseg = 1;
    p.seg[0] = row_major_seg(w.qg, 2 * hdp, 2 * hdp, 0, 0, 0);
    p.col_bias = q_bias;
    GemmOperandA a = {x_q, c, 0, 0};
    GemmOperandB b = {w_q_packed, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 128, "apb_cross_q_proj"));
  }
  {
    // key side: k position-major, v transposed per batch entry (keys contiguous)
    GemmParams p = {};
    p.n_extent = lk;
    p.o_extent = batch;
    p.batch = 1;
    p.n_cols = 2 * hdp;
    p.k_extent = c;
    p.nseg = 2;
    p.seg[0] = row_major_seg(w.kk, hdp, hdp, static_cast<long long>(lk) * hdp, 0, 0, 0);
    EpiSeg& sv = p.seg[1];
    sv = {};
    sv.col_begin = hdp;
    sv.ncols = hdp;
    sv.dst = w.vt;
    sv.s_col = lk;
    sv.s_n = 1;
    sv.s_o = static_cast<long long>(hdp) * lk;
    GemmOperandA a = {x_k, c, static_cast<long long>(lk) * c, 0};
    GemmOperandB b = {w_kv_packed, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 128, "apb_cross_kv_proj"));
  }
  {
    AttnParams p = {};
    p.batch = batch;
    p.heads = heads;
    p.lq = lq;
    p.lk = lk;
    p.d = d;
    p.dpad = dp;
    p.q = w.qg; p.ldq = 2 * hdp; p.q_col0 = 0;
    p.g = w.qg; p.ldg = 2 * hdp; p.g_col0 = hdp;
    p.k = w.kk; p.ldk = hdp; p.k_col0 = 0;
    p.vt = w.vt; p.ldv = lk;
    p.bias = pair_bias; p.ldb = lk; p.bias_div = bias_div; p.bias_mod = bias_mod; p.bias_head_major = bias_head_major;
    p.mask = mask;
    p.mask_lo_extent = 1;
    p.m_hi = lk;
    p.m_lo = 0;
    p.m_k = 1;
    p.out = w.og; p.ldo = c;
    p.tag = "apb_cross_attention";
    KFB_TRY(launch_attention(stream, p));
  }
  {
    GemmParams p = {};
    p.n_extent = static_cast<int>(gate_rows);
    p.o_extent = gate_reps;
    p.batch = 1;
    p.n_cols = c;
    p.k_extent = c;
    p.nseg = 1;
    p.seg[0] = row_major_seg(out, c, c, gate_rows * c, 0, out_dtype == KFB_FP32);
    p.col_bias = out_bias;
    p.resid = resid;
    if (out_gate != nullptr) {
      p.gate = static_cast<const __nv_bfloat16*>(out_gate);  // query row r uses logits row r % gate_rows
      p.g_col = 1;
      p.g_n = gate_ld;
      p.g_o = 0;
      p.g_b = 0;
    }
    GemmOperandA a = {w.og, c, gate_rows * c, 0};
    GemmOperandB b = {w_out, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "apb_cross_out_proj"));
  }
  return KFB_OK;
}

KFB_API size_t kfb_apb_window_workspace_bytes(int batch, int l, int c, int heads) {
  ApbCrossWs w;
  return carve_apb_cross(w, nullptr, batch, l, l, c, heads);
}

KFB_API int kfb_apb_window_fwd(const void* x_q, const void* x_k, const void* pair_bias, const unsigned char* mask,
                               const void* w_q_packed, const float* q_bias, const void* w_kv_packed, const void* w_out,
                               const float* out_bias, const void* out_gate, long long gate_rows, long long gate_ld, void* out,
                               const void* resid, void* workspace, size_t workspace_bytes, int batch, int l, int c, int heads, int bias_share,
                               int mask_share, int bias_head_major, int out_dtype, void* stream_) {
  KFB_CHECK_ARG(x_q && x_k && pair_bias && mask && w_q_packed && w_kv_packed && w_out && out && workspace,
                "apb_window: null pointer");
  KFB_CHECK_ARG(out_dtype == KFB_BF16 || out_dtype == KFB_FP32, "apb_window: dtype %d (bf16 or fp32 output, bf16 compute)", out_dtype);
  KFB_CHECK_ARG(batch >= 1 && l >= 32 && l % 32 == 0, "apb_window: %d atoms must be a positive multiple of 32", l);
  KFB_CHECK_ARG(heads >= 1 && c % heads == 0 && c % 8 == 0, "apb_window: c=%d heads=%d", c, heads);
  KFB_CHECK_ARG(bias_share >= 1 && batch % bias_share == 0 && mask_share >= 1 && batch % mask_share == 0 && bias_head_major >= 0,
                "apb_window: batch %d bias_share %d mask_share %d", batch, bias_share, mask_share);
  const int d = c / heads;
  KFB_CHECK_ARG(d % 8 == 0 && d >= 16 && d <= 32, "apb_window: head dim %d not in {16, 24, 32}", d);
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "apb_window: workspace must be 256-byte aligned");
  cudaStream_t stream = as_stream(stream_);
  const long long rows = static_cast<long long>(batch) * l;
  if (out_gate == nullptr || gate_rows <= 0) gate_rows = rows;
  if (gate_ld <= 0) gate_ld = c;
  KFB_CHECK_ARG(gate_ld >= c, "apb_window: gate row stride %lld below c=%d", gate_ld, c);
  KFB_CHECK_ARG(out_gate == nullptr || (gate_ld % 8 == 0 && (reinterpret_cast<uintptr_t>(out_gate) & 15) == 0),
                "apb_window: bf16 gate rows must start on 16-byte boundaries (pointer and row stride %lld)", gate_ld);
  KFB_CHECK_ARG(rows % gate_rows == 0 && gate_rows < (1ll << 31), "apb_window: %lld rows are not a multiple of gate_rows %lld", rows,
                gate_rows);
  const int gate_reps = static_cast<int>(rows / gate_rows);
  const int dp = dpad_of(d), hdp = heads * dp;
  ApbCrossWs w;
  const size_t need = carve_apb_cross(w, workspace, batch, l, l, c, heads);
  KFB_CHECK_ARG(workspace_bytes >= need, "apb_window: workspace %zu < %zu bytes", workspace_bytes, need);
  {
    GemmParams p = {};
    p.n_extent = static_cast<int>(rows);
    p.o_extent = 1;
    p.batch = 1;
    p.n_cols = 2 * hdp;
    p.k_extent = c;
    p.nseg = 1;
    p.seg[0] = row_major_seg(w.qg, 2 * hdp, 2 * hdp, 0, 0, 0);
    p.col_bias = q_bias;
    GemmOperandA a = {x_q, c, 0, 0};
    GemmOperandB b = {w_q_packed, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 128, "apb_window_q_proj"));
  }
  {
    // keys of the un-windowed atoms: k position-major, v transposed per sample (atoms contiguous)
    GemmParams p = {};
    p.n_extent = l;
    p.o_extent = batch;
    p.batch = 1;
    p.n_cols = 2 * hdp;
    p.k_extent = c;
    p.nseg = 2;
    p.seg[0] = row_major_seg(w.kk, hdp, hdp, static_cast<long long>(l) * hdp, 0, 0, 0);
    EpiSeg& sv = p.seg[1];
    sv = {};
    sv.col_begin = hdp;
    sv.ncols = hdp;
    sv.dst = w.vt;
    sv.s_col = l;
    sv.s_n = 1;
    sv.s_o = static_cast<long long>(hdp) * l;
    GemmOperandA a = {x_k, c, static_cast<long long>(l) * c, 0};
    GemmOperandB b = {w_kv_packed, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 128, "apb_window_kv_proj"));
  }
  {
    AttnParams p = {};
    p.batch = batch;
    p.heads = heads;
    p.lq = l;
    p.lk = l;
    p.d = d;
    p.dpad = dp;
    p.win = 1;
    p.q = w.qg; p.ldq = 2 * hdp; p.q_col0 = 0;
    p.g = w.qg; p.ldg = 2 * hdp; p.g_col0 = hdp;
    p.k = w.kk; p.ldk = hdp; p.k_col0 = 0;
    p.vt = w.vt; p.ldv = l;
    p.bias = pair_bias; p.ldb = 128; p.bias_div = bias_share; p.bias_mod = l / 32; p.bias_head_major = bias_head_major;
    p.mask = mask;
    p.mask_lo_extent = mask_share;   // batch entry b reads mask row b / mask_share
    p.m_hi = l;
    p.m_lo = 0;
    p.m_k = 1;
    p.out = w.og; p.ldo = c;
    p.tag = "apb_window_attention";
    KFB_TRY(launch_attention(stream, p));
  }
  {
    GemmParams p = {};
    p.n_extent = static_cast<int>(gate_rows);
    p.o_extent = gate_reps;
    p.batch = 1;
    p.n_cols = c;
    p.k_extent = c;
    p.nseg = 1;
    p.seg[0] = row_major_seg(out, c, c, gate_rows * c, 0, out_dtype == KFB_FP32);
    p.col_bias = out_bias;
    p.resid = resid;
    if (out_gate != nullptr) {
      p.gate = static_cast<const __nv_bfloat16*>(out_gate);  // row r uses logits row r % gate_rows
      p.g_col = 1;
      p.g_n = gate_ld;
      p.g_o = 0;
      p.g_b = 0;
    }
    GemmOperandA a = {w.og, c, gate_rows * c, 0};
    GemmOperandB b = {w_out, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "apb_window_out_proj"));
  }
  return KFB_OK;
}

}  // extern "C"
