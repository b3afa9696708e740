// Triangle multiplication (outgoing / incoming) as a sequence of sm_100a kernels.
//
//   phase "project"  (per position, local to a row shard)
//   1. LayerNorm_in                      x -> xn (bf16, position-major)             [HBM bound]
//   2. input projection + gate + mask    ab[ch] = (xn Wp^T) * sigmoid(xn Wg^T) * m  [tcgen05 GEMM, GLU epilogue,
//                                        stored CHANNEL-major so each channel is      channel-major TMA store]
//                                        a dense rows x N matrix
//   3. output gate logits                gl = xn Wg_out^T                            [tcgen05 GEMM]
//   phase "finish"
//   4. triangle contraction              t[ch] = A_ch * B_ch^T, batch over channels   [tcgen05 batched GEMM]
//   5. LayerNorm_out, channel-major in   t -> tn (bf16, position-major)             [HBM bound]
//   6. output projection * sigmoid(gl)   out = (tn Wp_out^T) * sigmoid(gl) (+ resid) [tcgen05 GEMM, gated epilogue]
//
// The incoming direction needs t[i,j] = sum_k a[k,i] b[k,j].  Instead of a second, MN-major contraction
// kernel, step 2 walks the pair tensor transposed (the TMA map of xn swaps its two position strides) so that
// it writes a^T and b^T; step 4 is then the very same K-major contraction for both directions.
//
// Row sharding across GPUs: a rank holds `rows` of the n token rows.  "project" runs on the shard, the caller
// all-gathers the b operand (every rank needs all rows j of b), and "finish" takes the gathered operand in the
// layout the collective leaves it in: rank after rank, each piece [channel][rows][n].
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

int check_shape(const char* what, int batch, int rows, int n, int c) {
  KFB_CHECK_ARG(batch >= 1 && n >= 8 && n % 8 == 0, "%s: N=%d must be a positive multiple of 8 (pad in the caller)", what, n);
  KFB_CHECK_ARG(rows >= 1 && rows <= n, "%s: rows=%d out of range for N=%d", what, rows, n);
  KFB_CHECK_ARG(c % 64 == 0 && c >= 64 && c <= 512, "%s: C=%d must be a multiple of 64 in [64, 512]", what, c);
  return KFB_OK;
}

// steps 1-3 on a (batch, rows, n, c) tensor.  transposed_walk writes a^T, b^T: ab[ch][b][column][row of the shard].
// x == nullptr: xn already holds the normalised input (a second call on the same tensor).
// parts > 1: only part `part` of the 2c operand channels (in packed order) is projected, into `ab` = that part's buffer.
int project(cudaStream_t stream, int transposed_walk, const void* x, const unsigned char* mask, const float* ln_w,
            const float* ln_b, const void* w_in_packed, const void* w_gout, __nv_bfloat16* xn, __nv_bfloat16* ab,
            __nv_bfloat16* gl, int batch, int rows, int n, int c, float eps, int dtype, int part = 0, int parts = 1) {
  const long long rn = static_cast<long long>(rows) * n;
  const long long pos = rn * batch;
  if (x != nullptr) KFB_TRY(launch_layernorm(stream, x, xn, ln_w, ln_b, pos, c, c, c, eps, dtype, KFB_BF16));
  if (w_in_packed != nullptr) {
    // ab[ch][b][o][n_]: o = row of the shard, n_ = position inside the row (swapped for the transposed walk)
    GemmParams p = {};
    p.n_extent = transposed_walk ? rows : n;
    p.o_extent = transposed_walk ? n : rows;
    p.batch = batch;
    p.n_cols = 4 * c / parts;
    p.k_extent = c;
    p.glu = GLU_SIGMOID;
    p.nseg = 1;
    EpiSeg& s = p.seg[0];
    s.col_begin = 0;
    s.ncols = 2 * c / parts;
    s.out_fp32 = 0;
    s.vec = 0;
    s.dst = ab;
    s.s_col = pos;
    s.s_n = 1;
    s.s_o = p.n_extent;
    s.s_b = rn;
    p.rowmask = mask;
    p.mask_segs = 1;
    p.m_b = rn;
    p.m_o = transposed_walk ? 1 : n;
    p.m_n = transposed_walk ? n : 1;
    GemmOperandA a = {xn, transposed_walk ? static_cast<long long>(n) * c : c,
                      transposed_walk ? c : static_cast<long long>(n) * c, rn * c};
    GemmOperandB b = {static_cast<const __nv_bfloat16*>(w_in_packed) + static_cast<long long>(part) * (4 * c / parts) * c, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 256, "trimul_in_proj"));
  }
  if (w_gout != nullptr) {
    GemmParams p = {};
    p.n_extent = static_cast<int>(pos);
    p.o_extent = 1;
    p.batch = 1;
    p.n_cols = c;
    p.k_extent = c;
    p.nseg = 1;
    p.seg[0] = row_major_seg(gl, c, c, 0, 0, 0);
    GemmOperandA a = {xn, c, 0, 0};
    GemmOperandB b = {w_gout, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "trimul_gate_proj"));
  }
  return KFB_OK;
}

// steps 4-6.  a: [c][batch][rows][n]; b: pieces of [c][batch][b_piece_rows][n], `b_piece_stride` elements apart.
int finish(cudaStream_t stream, const __nv_bfloat16* a, const __nv_bfloat16* b, int b_piece_rows, long long b_piece_stride,
           const __nv_bfloat16* gl, const float* ln_out_w, const float* ln_out_b, const void* w_pout, __nv_bfloat16* t,
           __nv_bfloat16* tn, void* out, const void* resid, int batch, int rows, int n, int c, float eps, int dtype) {
  const long long rn = static_cast<long long>(rows) * n;
  const long long pos = rn * batch;
  if (a != nullptr) {
    // t[ch*B+b][i][j] = sum_k A[i][k] B[j][k]
    GemmParams p = {};
    p.n_extent = rows;
    p.o_extent = 1;
    p.batch = c * batch;
    p.n_cols = n;
    p.k_extent = n;
    p.b_batched = 1;
    p.nseg = 1;
    p.seg[0] = row_major_seg(t, n, n, 0, rn, 0);
    GemmOperandA oa = {a, n, 0, rn};
    GemmOperandB ob = {b, n, static_cast<long long>(b_piece_rows) * n};
    int force_bn = 0;
    if (b_piece_rows != n) {
      ob.col_inner = b_piece_rows;
      ob.s_col_hi = b_piece_stride;
      force_bn = b_piece_rows % 256 == 0 ? 256 : (b_piece_rows % 128 == 0 ? 128 : 64);
    }
    KFB_TRY(launch_gemm_bf16(stream, oa, ob, p, force_bn, "trimul_contraction"));
  }
  // LayerNorm_out folded into the output projection: the GEMM reads t as it lies (channel-major, read MN-major), the
  // epilogue applies the per-position statistics.  The scratch buffer tn holds the folded weights and the statistics.
  const bool fold = (c % kBK == 0) && (pos % 8 == 0) &&
                    pos * static_cast<long long>(c) * 2 >= static_cast<long long>(c) * c * 2 + 256 + 2ll * c * 4 + 256 + pos * 8;
  if (fold) {
    uint8_t* base = reinterpret_cast<uint8_t*>(tn);
    __nv_bfloat16* wf = reinterpret_cast<__nv_bfloat16*>(base);
    float* s1 = reinterpret_cast<float*>(base + align_up(static_cast<size_t>(c) * c * 2, 256));
    float* s0 = s1 + c;
    float2* stats = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(s1) + align_up(static_cast<size_t>(2) * c * 4, 256));
    KFB_TRY(launch_ln_fold_weights(stream, static_cast<const __nv_bfloat16*>(w_pout), ln_out_w, ln_out_b, wf, s1, s0, c, c));
    KFB_TRY(launch_cm_stats(stream, t, stats, pos, c, pos, eps));
    GemmParams p = {};
    p.n_extent = static_cast<int>(pos);
    p.o_extent = 1;
    p.batch = 1;
    p.n_cols = c;
    p.k_extent = c;
    p.nseg = 1;
    p.seg[0] = row_major_seg(out, c, c, 0, 0, dtype == KFB_FP32);
    p.gate = gl;
    p.g_col = 1;
    p.g_n = c;
    p.resid = resid;
    p.row_stats = stats;
    p.col_s1 = s1;
    p.col_s0 = s0;
    GemmOperandA oa = {t, 1, 0, 0};
    oa.s_k = pos;
    GemmOperandB ob = {wf, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, oa, ob, p, 0, "trimul_out_proj"));
    return KFB_OK;
  }
  KFB_TRY(launch_layernorm_cm(stream, t, tn, ln_out_w, ln_out_b, batch, rn, c, pos, rn, eps, KFB_BF16));
  {
    GemmParams p = {};
    p.n_extent = static_cast<int>(pos);
    p.o_extent = 1;
    p.batch = 1;
    p.n_cols = c;
    p.k_extent = c;
    p.nseg = 1;
    p.seg[0] = row_major_seg(out, c, c, 0, 0, dtype == KFB_FP32);
    p.gate = gl;
    p.g_col = 1;
    p.g_n = c;
    p.resid = resid;
    GemmOperandA oa = {tn, c, 0, 0};
    GemmOperandB ob = {w_pout, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, oa, ob, p, 0, "trimul_out_proj"));
  }
  return KFB_OK;
}

// ------------------------------------------------------------------------------------------------
// fp32-accurate variant (KFB_FP32_PRECISE): same six steps, every GEMM operand stored as the bf16 triple split
// concatenated along K, fp32 intermediates (gate logits, contraction result).
// ------------------------------------------------------------------------------------------------
struct TrimulWsPrecise {
  __nv_bfloat16 *xn6, *ab6;
  float *gl, *t;
};
size_t carve_precise(TrimulWsPrecise& w, void* base, int batch, int n, int c) {
  Carver cv(base);
  const size_t pos = static_cast<size_t>(batch) * n * n;
  w.xn6 = cv.take<__nv_bfloat16>(pos * 6 * c);  // reused as tn6
  w.ab6 = cv.take<__nv_bfloat16>(pos * 6 * 2 * c);
  w.gl = cv.take<float>(pos * c);
  w.t = cv.take<float>(pos * c);
  return cv.off;
}

int trimul_precise(cudaStream_t stream, int incoming, const void* x, const unsigned char* mask, const float* ln_in_w,
                   const float* ln_in_b, const void* w_in6, const void* w_gout6, const float* ln_out_w, const float* ln_out_b,
                   const void* w_pout6, void* out, const void* resid, const TrimulWsPrecise& w, int batch, int n, int c,
                   float eps) {
  const long long nn = static_cast<long long>(n) * n;
  const long long pos = nn * batch;
  KFB_TRY(launch_layernorm_split(stream, static_cast<const float*>(x), w.xn6, ln_in_w, ln_in_b, pos, c, c, eps, 1));
  {
    // a -> split pattern 1, b -> pattern 2, both channel-major with the six parts along k: ab6[ch][b][o][6n]
    GemmParams p = {};
    p.n_extent = n;
    p.o_extent = n;
    p.batch = batch;
    p.n_cols = 4 * c;
    p.k_extent = 6 * c;
    p.glu = GLU_SIGMOID;
    p.precise = 1;
    p.nseg = 2;
    for (int i = 0; i < 2; ++i) {
      EpiSeg& s = p.seg[i];
      s = {};
      s.col_begin = i * c;
      s.ncols = c;
      s.dst = w.ab6 + static_cast<long long>(i) * c * pos * 6;
      s.s_col = 6 * pos;
      s.s_n = 1;
      s.s_o = 6ll * n;
      s.s_b = 6 * nn;
      s.split = i + 1;
      s.s_part = n;
    }
    p.rowmask = mask;
    p.mask_segs = 3;
    p.m_b = nn;
    p.m_o = incoming ? 1 : n;
    p.m_n = incoming ? n : 1;
    const long long c6 = 6ll * c;
    GemmOperandA a = {w.xn6, incoming ? n * c6 : c6, incoming ? c6 : n * c6, nn * c6};
    GemmOperandB b = {w_in6, c6, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 128, "trimul_in_proj_precise"));
  }
  {
    GemmParams p = {};
    p.n_extent = static_cast<int>(pos);
    p.o_extent = 1;
    p.batch = 1;
    p.n_cols = c;
    p.k_extent = 6 * c;
    p.precise = 1;
    p.nseg = 1;
    p.seg[0] = row_major_seg(w.gl, c, c, 0, 0, 1);
    GemmOperandA a = {w.xn6, 6ll * c, 0, 0};
    GemmOperandB b = {w_gout6, 6ll * c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "trimul_gate_proj_precise"));
  }
  {
    GemmParams p = {};
    p.n_extent = n;
    p.o_extent = 1;
    p.batch = c * batch;
    p.n_cols = n;
    p.k_extent = 6 * n;
    p.b_batched = 1;
    p.precise = 1;
    p.nseg = 1;
    p.seg[0] = row_major_seg(w.t, n, n, 0, nn, 1);
    GemmOperandA a = {w.ab6, 6ll * n, 0, 6 * nn};
    GemmOperandB b = {w.ab6 + static_cast<long long>(c) * pos * 6, 6ll * n, 6 * nn};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "trimul_contraction_precise"));
  }
  __nv_bfloat16* tn6 = w.xn6;
  KFB_TRY(launch_layernorm_cm(stream, w.t, tn6, ln_out_w, ln_out_b, batch, nn, c, pos, nn, eps, KFB_FP32, 1));
  {
    GemmParams p = {};
    p.n_extent = static_cast<int>(pos);
    p.o_extent = 1;
    p.batch = 1;
    p.n_cols = c;
    p.k_extent = 6 * c;
    p.precise = 1;
    p.nseg = 1;
    p.seg[0] = row_major_seg(out, c, c, 0, 0, 1);
    p.gate = reinterpret_cast<const __nv_bfloat16*>(w.gl);  // fp32 logits in precise mode
    p.g_col = 1;
    p.g_n = c;
    p.resid = resid;
    GemmOperandA a = {tn6, 6ll * c, 0, 0};
    GemmOperandB b = {w_pout6, 6ll * c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "trimul_out_proj_precise"));
  }
  return KFB_OK;
}

}  // namespace

extern "C" {

KFB_API size_t kfb_trimul_workspace_bytes_precise(int batch, int n, int c) {
  TrimulWsPrecise w;
  return carve_precise(w, nullptr, batch, n, c);
}

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
  KFB_TRY(check_shape("trimul", batch, n, n, c));
  if (dtype == KFB_FP32_PRECISE) {
    KFB_CHECK_ARG(c <= 256, "trimul: the fp32-accurate mode supports at most 256 channels");
    TrimulWsPrecise wp;
    const size_t need_p = carve_precise(wp, workspace, batch, n, c);
    KFB_CHECK_ARG(workspace_bytes >= need_p, "trimul: workspace %zu < %zu bytes", workspace_bytes, need_p);
    KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "trimul: workspace must be 256-byte aligned");
    return trimul_precise(as_stream(stream_), incoming, x, mask, ln_in_w, ln_in_b, w_in_packed, w_gout, ln_out_w, ln_out_b,
                          w_pout, out, resid, wp, batch, n, c, eps);
  }
  TrimulWs w;
  const size_t need = carve(w, workspace, batch, n, c);
  KFB_CHECK_ARG(workspace_bytes >= need, "trimul: workspace %zu < %zu bytes", workspace_bytes, need);
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "trimul: workspace must be 256-byte aligned");
  cudaStream_t stream = as_stream(stream_);
  const long long pos = static_cast<long long>(batch) * n * n;
  KFB_TRY(project(stream, incoming, x, mask, ln_in_w, ln_in_b, w_in_packed, w_gout, w.xn, w.ab, w.gl, batch, n, n, c, eps, dtype));
  return finish(stream, w.ab, w.ab + static_cast<long long>(c) * pos, n, 0, w.gl, ln_out_w, ln_out_b, w_pout, w.t, w.xn, out,
                resid, batch, n, n, c, eps, dtype);
}

KFB_API int kfb_trimul_project(const void* x, const unsigned char* mask, const float* ln_in_w, const float* ln_in_b,
                               const void* w_in_packed, const void* w_gout, void* xn_scratch, void* ab_out, void* gl_out,
                               int batch, int rows, int n, int c, int transposed, int part, int parts, float eps, int dtype,
                               void* stream_) {
  KFB_CHECK_ARG(xn_scratch, "trimul_project: null pointer");
  KFB_CHECK_ARG(parts >= 1 && part >= 0 && part < parts && (4 * c) % (256 * parts) == 0,
                "trimul_project: part %d of %d needs 4C=%d to split into whole 256-column tiles", part, parts, 4 * c);
  KFB_CHECK_ARG((w_in_packed == nullptr) == (ab_out == nullptr) && (w_gout == nullptr) == (gl_out == nullptr),
                "trimul_project: each weight needs its output buffer and vice versa");
  KFB_CHECK_ARG(w_in_packed == nullptr || mask != nullptr, "trimul_project: the input projection needs the mask");
  KFB_CHECK_ARG(is_dtype(dtype), "trimul_project: bad dtype %d", dtype);
  KFB_TRY(check_shape("trimul_project", batch, rows, n, c));
  return project(as_stream(stream_), transposed ? 1 : 0, x, mask, ln_in_w, ln_in_b, w_in_packed, w_gout, static_cast<__nv_bfloat16*>(xn_scratch),
                 static_cast<__nv_bfloat16*>(ab_out), static_cast<__nv_bfloat16*>(gl_out), batch, rows, n, c, eps, dtype, part,
                 parts);
}

// The contraction alone, on `cpart` channels: t[ch][i][j] = sum_k a[ch][i][k] b[ch][j][k] with b in gathered pieces (as in
// kfb_trimul_finish).  Lets the caller contract one half of the channels while the other half's operand is still in flight;
// kfb_trimul_finish is then called with a = b = NULL.
KFB_API int kfb_trimul_contract(const void* a, const void* b_gathered, int b_piece_rows, long long b_piece_stride, void* t, int rows,
                                int n, int cpart, void* stream_) {
  KFB_CHECK_ARG(a && b_gathered && t && cpart >= 1, "trimul_contract: null pointer");
  KFB_CHECK_ARG(rows >= 1 && rows <= n && n % 8 == 0, "trimul_contract: rows=%d N=%d", rows, n);
  KFB_CHECK_ARG(b_piece_rows >= 64 && n % b_piece_rows == 0 && b_piece_rows % 64 == 0 && b_piece_stride % 8 == 0,
                "trimul_contract: pieces of %d rows (multiple of 64 dividing N=%d), stride %lld", b_piece_rows, n, b_piece_stride);
  const long long rn = static_cast<long long>(rows) * n;
  GemmParams p = {};
  p.n_extent = rows;
  p.o_extent = 1;
  p.batch = cpart;
  p.n_cols = n;
  p.k_extent = n;
  p.b_batched = 1;
  p.nseg = 1;
  p.seg[0] = row_major_seg(t, n, n, 0, rn, 0);
  GemmOperandA oa = {a, n, 0, rn};
  GemmOperandB ob = {b_gathered, n, static_cast<long long>(b_piece_rows) * n};
  int force_bn = 0;
  if (b_piece_rows != n) {
    ob.col_inner = b_piece_rows;
    ob.s_col_hi = b_piece_stride;
    force_bn = b_piece_rows % 256 == 0 ? 256 : (b_piece_rows % 128 == 0 ? 128 : 64);
  }
  return launch_gemm_bf16(as_stream(stream_), oa, ob, p, force_bn, "trimul_contraction");
}

KFB_API int kfb_trimul_finish(const void* a, const void* b_gathered, int b_piece_rows, long long b_piece_stride,
                              const void* gl, const float* ln_out_w, const float* ln_out_b, const void* w_pout,
                              void* t_scratch, void* tn_scratch, void* out, const void* resid, int rows, int n, int c,
                              float eps, int dtype, void* stream_) {
  KFB_CHECK_ARG(gl && w_pout && t_scratch && tn_scratch && out, "trimul_finish: null pointer");
  KFB_CHECK_ARG((a == nullptr) == (b_gathered == nullptr), "trimul_finish: pass both operands, or neither when t_scratch "
                "already holds the contraction result");
  KFB_CHECK_ARG(is_dtype(dtype), "trimul_finish: bad dtype %d", dtype);
  KFB_TRY(check_shape("trimul_finish", 1, rows, n, c));
  KFB_CHECK_ARG(b_piece_rows >= 64 && n % b_piece_rows == 0 && b_piece_rows % 64 == 0 && b_piece_stride % 8 == 0,
                "trimul_finish: pieces of %d rows (multiple of 64 dividing N=%d), stride %lld", b_piece_rows, n, b_piece_stride);
  return finish(as_stream(stream_), static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b_gathered),
                b_piece_rows, b_piece_stride, static_cast<const __nv_bfloat16*>(gl), ln_out_w, ln_out_b, w_pout,
                static_cast<__nv_bfloat16*>(t_scratch), static_cast<__nv_bfloat16*>(tn_scratch), out, resid, 1, rows, n, c, eps,
                dtype);
}

// Channel-sharded contraction.  After an all-to-all of the ranks' projections this rank holds ALL pair rows of a and b
// for `cl` of the channels: ab_recv [world (source rank q)][2 (a, b)][cl][rows][n], rows q*rows .. q*rows+rows-1 of the pair
// tensor coming from rank q.  Result t_send [world (q)][cl][rows][n]: the rows of t that belong to rank q, laid out for
// the all-to-all back (after which every rank holds t [c][rows][n] for its own rows, channel-major).
// incoming != 0: the ranks projected with the transposed walk, ab_recv is [world (q)][2][cl][n][rows] holding
// a[k = q*rows + k_q][i] at [i][k_q]; t[i][j] = sum_k a[k][i] b[k][j] is then a K-major product whose K lies in `world` pieces.
KFB_API int kfb_trimul_contract_cs(const void* ab_recv, void* t_send, int world, int rows, int n, int cl, int incoming,
                                   void* stream_) {
  KFB_CHECK_ARG(ab_recv && t_send, "trimul_contract_cs: null pointer");
  KFB_CHECK_ARG(world >= 1 && rows >= 64 && rows % 64 == 0 && static_cast<long long>(world) * rows == n && cl >= 1,
                "trimul_contract_cs: world %d x rows %d (multiple of 64) must equal N=%d; channels %d", world, rows, n, cl);
  const long long rn = static_cast<long long>(rows) * n;
  const __nv_bfloat16* a = static_cast<const __nv_bfloat16*>(ab_recv);
  GemmParams p = {};
  p.n_extent = rows;     // pair row inside the source rank's shard
  p.o_extent = world;    // source rank
  p.batch = cl;          // channel
  p.n_cols = n;
  p.k_extent = n;
  p.b_batched = 1;
  p.nseg = 1;
  p.seg[0] = row_major_seg(t_send, n, n, static_cast<long long>(cl) * rn, rn, 0);
  if (incoming) {
    GemmOperandA oa = {a, rows, static_cast<long long>(rows) * rows, rn};
    oa.k_inner = rows;
    oa.s_k_hi = 2ll * cl * rn;
    GemmOperandB ob = {a + static_cast<long long>(cl) * rn, rows, rn};
    ob.k_inner = rows;
    ob.s_k_hi = 2ll * cl * rn;
    const int bn = n % 256 == 0 ? 256 : (n % 128 == 0 ? 128 : 64);
    return launch_gemm_bf16(as_stream(stream_), oa, ob, p, bn, "trimul_contraction");
  }
  GemmOperandA oa = {a, n, 2ll * cl * rn, rn};
  GemmOperandB ob = {a + static_cast<long long>(cl) * rn, n, rn};
  ob.col_inner = rows;
  ob.s_col_hi = 2ll * cl * rn;
  const int force_bn = rows % 256 == 0 ? 256 : (rows % 128 == 0 ? 128 : 64);
  return launch_gemm_bf16(as_stream(stream_), oa, ob, p, force_bn, "trimul_contraction");
}

}  // extern "C"
