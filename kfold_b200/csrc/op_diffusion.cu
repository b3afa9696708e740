// Conditioned (diffusion) variants: adaptive LayerNorm and the conditioned transition block.
//
// The conditioning tensor s is shared by the diffusion samples, so everything derived from it (the AdaLN
// gate / shift, the output gates) is computed once per token by small GEMMs in the caller and passed in as
// bf16 logits; the kernels here broadcast those rows over the samples.
#include "ops_common.cuh"

using namespace kfb;

extern "C" {

// y = sigmoid(gv[:, :c]) * LayerNorm(a) + gv[:, c:]
KFB_API int kfb_adaln_fwd(const void* a, const void* gate_shift, long long gate_shift_ld, void* out, long long rows, int c,
                          int samples, int l, float eps, int in_dtype, void* stream) {
  KFB_CHECK_ARG(a && gate_shift && out, "adaln: null pointer");
  KFB_CHECK_ARG(is_dtype(in_dtype), "adaln: bad dtype %d", in_dtype);
  // KFB_FP32_PRECISE: a, gate_shift and out are all fp32
  return launch_adaln(as_stream(stream), a, out, gate_shift, rows, c, samples, l, eps, in_dtype,
                      in_dtype == KFB_FP32_PRECISE ? KFB_FP32 : KFB_BF16, gate_shift_ld);
}

// y = x W^T (+ bias) at fp32 accuracy: x fp32 [rows, k], w6 the bf16 triple split of W [n, 6k], out fp32 [rows, n]
KFB_API size_t kfb_linear_fp32_workspace_bytes(long long rows, int k) {
  return align_up(static_cast<size_t>(rows) * 6 * k * sizeof(__nv_bfloat16), 256);
}

KFB_API int kfb_linear_fp32(const void* x, const void* w6, const float* bias, void* out, void* workspace,
                            size_t workspace_bytes, long long rows, int n, int k, void* stream_) {
  KFB_CHECK_ARG(x && w6 && out && workspace, "linear_fp32: null pointer");
  KFB_CHECK_ARG(rows >= 1 && rows < (1ll << 31) && n >= 1 && k >= 8 && k % 8 == 0, "linear_fp32: rows %lld n %d k %d", rows, n, k);
  KFB_CHECK_ARG(workspace_bytes >= kfb_linear_fp32_workspace_bytes(rows, k), "linear_fp32: workspace too small");
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "linear_fp32: workspace must be 256-byte aligned");
  cudaStream_t stream = as_stream(stream_);
  __nv_bfloat16* x6 = static_cast<__nv_bfloat16*>(workspace);
  KFB_TRY(launch_layernorm_split(stream, static_cast<const float*>(x), x6, nullptr, nullptr, rows, k, k, 0.f, 0));
  GemmParams p = {};
  p.n_extent = static_cast<int>(rows);
  p.o_extent = 1;
  p.batch = 1;
  p.n_cols = n;
  p.k_extent = 6 * k;
  p.precise = 1;
  p.nseg = 1;
  p.seg[0] = row_major_seg(out, n, n, 0, 0, 1);
  p.col_bias = bias;
  GemmOperandA a = {x6, 6ll * k, 0, 0};
  GemmOperandB b = {w6, 6ll * k, 0};
  return launch_gemm_bf16(stream, a, b, p, 0, "linear_fp32");
}

// out = LayerNorm(x) W^T (+ bias) (+ resid) at fp32 accuracy; `normalise` == 0 skips the LayerNorm
KFB_API int kfb_ln_linear_fp32(const void* x, const float* ln_w, const float* ln_b, const void* w6, const float* bias,
                               const void* resid, void* out, void* workspace, size_t workspace_bytes, long long rows, int n, int k,
                               float eps, int normalise, void* stream_) {
  KFB_CHECK_ARG(x && w6 && out && workspace, "ln_linear_fp32: null pointer");
  KFB_CHECK_ARG(rows >= 1 && rows < (1ll << 31) && n >= 1 && k >= 8 && k % 8 == 0, "ln_linear_fp32: rows %lld n %d k %d", rows, n, k);
  KFB_CHECK_ARG(workspace_bytes >= kfb_linear_fp32_workspace_bytes(rows, k), "ln_linear_fp32: workspace too small");
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "ln_linear_fp32: workspace must be 256-byte aligned");
  cudaStream_t stream = as_stream(stream_);
  __nv_bfloat16* x6 = static_cast<__nv_bfloat16*>(workspace);
  KFB_TRY(launch_layernorm_split(stream, static_cast<const float*>(x), x6, normalise ? ln_w : nullptr, normalise ? ln_b : nullptr, rows,
                                 k, k, eps, normalise ? 1 : 0));
  GemmParams p = {};
  p.n_extent = static_cast<int>(rows);
  p.o_extent = 1;
  p.batch = 1;
  p.n_cols = n;
  p.k_extent = 6 * k;
  p.precise = 1;
  p.nseg = 1;
  p.seg[0] = row_major_seg(out, n, n, 0, 0, 1);
  p.col_bias = bias;
  p.resid = resid;
  GemmOperandA a = {x6, 6ll * k, 0, 0};
  GemmOperandB b = {w6, 6ll * k, 0};
  return launch_gemm_bf16(stream, a, b, p, 0, "ln_linear_fp32");
}

KFB_API size_t kfb_cond_transition_workspace_bytes_precise(long long rows, int c, int hidden) {
  return align_up(static_cast<size_t>(rows) * 6 * c * 2, 256) + align_up(static_cast<size_t>(rows) * 6 * hidden * 2, 256);
}

KFB_API size_t kfb_cond_transition_workspace_bytes(long long rows, int hidden) {
  return align_up(static_cast<size_t>(rows) * hidden * sizeof(__nv_bfloat16), 256);
}

// out = sigmoid(gate[s(r)]) * (silu(u_a) * u_b) W_out^T  (+ resid),  [u_a, u_b] = x W_swiglu^T,  x already AdaLN-normalised
KFB_API int kfb_cond_transition_fwd(const void* x_normed, const void* w_swiglu_packed, const void* w_out,
                                    const void* out_gate, long long gate_ld, void* out, const void* resid, void* workspace,
                                    size_t workspace_bytes, long long rows, int c, int hidden, int samples, int l, int dtype,
                                    void* stream_) {
  KFB_CHECK_ARG(x_normed && w_swiglu_packed && w_out && out_gate && out && workspace, "cond_transition: null pointer");
  if (gate_ld <= 0) gate_ld = c;
  KFB_CHECK_ARG(gate_ld >= c, "cond_transition: gate row stride %lld below c=%d", gate_ld, c);
  KFB_CHECK_ARG(dtype == KFB_FP32_PRECISE || (gate_ld % 8 == 0 && (reinterpret_cast<uintptr_t>(out_gate) & 15) == 0),
                "cond_transition: bf16 gate rows must start on 16-byte boundaries (pointer and row stride %lld)", gate_ld);
  KFB_CHECK_ARG(is_dtype(dtype), "cond_transition: bad dtype %d", dtype);
  KFB_CHECK_ARG(rows >= 1 && rows < (1ll << 31) && samples >= 1 && l >= 1 && rows % (static_cast<long long>(samples) * l) == 0,
                "cond_transition: rows %lld samples %d l %d", rows, samples, l);
  KFB_CHECK_ARG(c % 8 == 0 && hidden % 128 == 0, "cond_transition: c=%d (multiple of 8), hidden=%d (multiple of 128)", c, hidden);
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "cond_transition: workspace must be 256-byte aligned");
  cudaStream_t stream = as_stream(stream_);
  if (dtype == KFB_FP32_PRECISE) {
    // x_normed, out_gate (logits), out and resid are fp32; the weights are bf16 triple splits
    KFB_CHECK_ARG(workspace_bytes >= kfb_cond_transition_workspace_bytes_precise(rows, c, hidden),
                  "cond_transition: workspace too small");
    Carver cv(workspace);
    __nv_bfloat16* x6 = cv.take<__nv_bfloat16>(static_cast<size_t>(rows) * 6 * c);
    __nv_bfloat16* h6 = cv.take<__nv_bfloat16>(static_cast<size_t>(rows) * 6 * hidden);
    KFB_TRY(launch_layernorm_split(stream, static_cast<const float*>(x_normed), x6, nullptr, nullptr, rows, c, c, 0.f, 0));
    {
      GemmParams p = {};
      p.n_extent = static_cast<int>(rows);
      p.o_extent = 1;
      p.batch = 1;
      p.n_cols = 2 * hidden;
      p.k_extent = 6 * c;
      p.glu = GLU_SWIGLU;
      p.precise = 1;
      p.nseg = 1;
      p.seg[0] = row_major_seg(h6, hidden, 6ll * hidden, 0, 0, 0);
      p.seg[0].vec = 0;
      p.seg[0].split = 1;
      p.seg[0].s_part = hidden;
      GemmOperandA a = {x6, 6ll * c, 0, 0};
      GemmOperandB b = {w_swiglu_packed, 6ll * c, 0};
      KFB_TRY(launch_gemm_bf16(stream, a, b, p, 128, "cond_transition_swiglu_precise"));
    }
    const int groups = static_cast<int>(rows / (static_cast<long long>(samples) * l));
    GemmParams p = {};
    p.n_extent = l;
    p.o_extent = samples;
    p.batch = groups;
    p.n_cols = c;
    p.k_extent = 6 * hidden;
    p.precise = 1;
    p.nseg = 1;
    const long long lc = static_cast<long long>(l) * c, lh6 = static_cast<long long>(l) * 6 * hidden;
    p.seg[0] = row_major_seg(out, c, c, lc, lc * samples, 1);
    p.resid = resid;
    p.gate = static_cast<const __nv_bfloat16*>(out_gate);  // fp32 logits in this mode
    p.g_col = 1;
    p.g_n = gate_ld;
    p.g_o = 0;
    p.g_b = l * gate_ld;
    GemmOperandA a = {h6, 6ll * hidden, lh6, lh6 * samples};
    GemmOperandB b = {w_out, 6ll * hidden, 0};
    return launch_gemm_bf16(stream, a, b, p, 0, "cond_transition_out_precise");
  }
  KFB_CHECK_ARG(workspace_bytes >= kfb_cond_transition_workspace_bytes(rows, hidden), "cond_transition: workspace too small");
  __nv_bfloat16* h = static_cast<__nv_bfloat16*>(workspace);
  {
    GemmParams p = {};
    p.n_extent = static_cast<int>(rows);
    p.o_extent = 1;
    p.batch = 1;
    p.n_cols = 2 * hidden;
    p.k_extent = c;
    p.glu = GLU_SWIGLU;
    p.nseg = 1;
    p.seg[0] = row_major_seg(h, hidden, hidden, 0, 0, 0);
    GemmOperandA a = {x_normed, c, 0, 0};
    GemmOperandB b = {w_swiglu_packed, c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 256, "cond_transition_swiglu"));
  }
  {
    const int groups = static_cast<int>(rows / (static_cast<long long>(samples) * l));
    GemmParams p = {};
    p.n_extent = l;
    p.o_extent = samples;
    p.batch = groups;
    p.n_cols = c;
    p.k_extent = hidden;
    p.nseg = 1;
    const long long lc = static_cast<long long>(l) * c, lh = static_cast<long long>(l) * hidden;
    p.seg[0] = row_major_seg(out, c, c, lc, lc * samples, dtype == KFB_FP32);
    p.resid = resid;
    p.gate = static_cast<const __nv_bfloat16*>(out_gate);
    p.g_col = 1;
    p.g_n = gate_ld;
    p.g_o = 0;
    p.g_b = l * gate_ld;
    GemmOperandA a = {h, hidden, lh, lh * samples};
    GemmOperandB b = {w_out, hidden, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "cond_transition_out"));
  }
  return KFB_OK;
}

KFB_API int kfb_window_bias_fwd(const void* z, const float* ln_w, const float* ln_b, const void* w, void* bias_out,
                                long long positions, int c, int heads, float eps, int normalise, int dtype, void* stream_) {
  KFB_CHECK_ARG(z && w && bias_out, "window_bias: null pointer");
  KFB_CHECK_ARG(is_dtype(dtype), "window_bias: bad dtype %d", dtype);
  KFB_CHECK_ARG(positions >= 0 && heads >= 1, "window_bias: positions %lld heads %d", positions, heads);
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(z) & 15) == 0, "window_bias: z must be 16-byte aligned");
  return launch_window_bias(as_stream(stream_), z, ln_w, ln_b, w, bias_out, positions, c, heads, eps, normalise,
                            dtype == KFB_FP32_PRECISE ? KFB_FP32 : dtype);
}

}  // extern "C"
