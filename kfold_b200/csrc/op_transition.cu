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

KFB_API size_t kfb_transition_workspace_bytes_precise(long long rows, int c, int hidden) {
  return align_up(static_cast<size_t>(rows) * 6 * c * 2, 256) + align_up(static_cast<size_t>(rows) * 6 * hidden * 2, 256);
}

// fp32-accurate transition: every operand is the bf16 triple split, concatenated along K (see kfold_b200.h)
static int transition_precise(cudaStream_t stream, const void* x, const float* ln_w, const float* ln_b, const void* w_swiglu6,
                              const void* w_out6, void* out, const void* resid, void* workspace, long long rows, int c,
                              int hidden, float eps) {
  Carver cv(workspace);
  __nv_bfloat16* xn6 = cv.take<__nv_bfloat16>(static_cast<size_t>(rows) * 6 * c);
  __nv_bfloat16* h6 = cv.take<__nv_bfloat16>(static_cast<size_t>(rows) * 6 * hidden);
  KFB_TRY(launch_layernorm_split(stream, static_cast<const float*>(x), xn6, ln_w, ln_b, rows, c, c, eps, 1));
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
    GemmOperandA a = {xn6, 6ll * c, 0, 0};
    GemmOperandB b = {w_swiglu6, 6ll * c, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 128, "transition_swiglu_precise"));
  }
  {
    GemmParams p = {};
    p.n_extent = static_cast<int>(rows);
    p.o_extent = 1;
    p.batch = 1;
    p.n_cols = c;
    p.k_extent = 6 * hidden;
    p.precise = 1;
    p.nseg = 1;
    p.seg[0] = row_major_seg(out, c, c, 0, 0, 1);
    p.resid = resid;
    GemmOperandA a = {h6, 6ll * hidden, 0, 0};
    GemmOperandB b = {w_out6, 6ll * hidden, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "transition_out_precise"));
  }
  return KFB_OK;
}

KFB_API int kfb_transition_fwd(const void* x, const float* ln_w, const float* ln_b, const void* w_swiglu_packed,
                               const void* w_out, void* out, const void* resid, void* workspace, size_t workspace_bytes,
                               long long rows, int c, int hidden, float eps, int dtype, void* stream_) {
  KFB_CHECK_ARG(x && w_swiglu_packed && w_out && out && workspace, "transition: null pointer");
  KFB_CHECK_ARG(is_dtype(dtype), "transition: bad dtype %d", dtype);
  KFB_CHECK_ARG(rows >= 1 && rows < (1ll << 31), "transition: rows %lld", rows);
  KFB_CHECK_ARG(c % 8 == 0 && hidden % 128 == 0, "transition: c=%d (multiple of 8), hidden=%d (multiple of 128)", c, hidden);
  if (dtype == KFB_FP32_PRECISE) {
    KFB_CHECK_ARG(workspace_bytes >= kfb_transition_workspace_bytes_precise(rows, c, hidden), "transition: workspace too small");
    KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "transition: workspace must be 256-byte aligned");
    return transition_precise(as_stream(stream_), x, ln_w, ln_b, w_swiglu_packed, w_out, out, resid, workspace, rows, c, hidden,
                              eps);
  }
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
    p.seg[0] = row_major_seg(out, c, c, 0, 0, is_fp32_io(dtype));
    p.resid = resid;
    GemmOperandA a = {w.h, hidden, 0, 0};
    GemmOperandB b = {w_out, hidden, 0};
    KFB_TRY(launch_gemm_bf16(stream, a, b, p, 0, "transition_out"));
  }
  return KFB_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Transition without a caller-provided workspace.
//
// Some hosts of this library cannot hand over scratch memory: a serving process whose device pool
// was sized and frozen at start-up, or a plugin callback that is not allowed to call cudaMalloc
// (the call synchronises the whole device and would stall every other stream of the process).
// For them the two temporaries of the transition (the normalised input and the SwiGLU hidden
// activations) live in the fixed device array below instead.  Every GPU that loads the library
// carries these 8 MiB until the process exits.
// ------------------------------------------------------------------------------------------------
#include <mutex>

static constexpr size_t kStaticScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_transition_scratch[kStaticScratchBytes];

namespace {
// Device address of g_transition_scratch per device ordinal.  In host code the array's name is only
// a handle for the runtime, not an address a kernel could use; cudaGetSymbolAddress translates it
// for the device that is current at the time of the call.
std::mutex g_scratch_mu;
void* g_scratch_ptr[64] = {};

int static_scratch(void** out) {
  int dev = 0;
  KFB_CUDA(cudaGetDevice(&dev));
  KFB_CHECK_ARG(dev >= 0 && dev < 64, "transition_static: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    KFB_CUDA(cudaGetSymbolAddress(&p, g_transition_scratch));
    KFB_CHECK_ARG(p != nullptr && (reinterpret_cast<uintptr_t>(p) & 255) == 0, "transition_static: bad scratch address %p", p);
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return KFB_OK;
}
}  // namespace

extern "C" {

KFB_API size_t kfb_transition_static_max_bytes(void) { return kStaticScratchBytes; }

KFB_API int kfb_transition_fwd_static(const void* x, const float* ln_w, const float* ln_b, const void* w_swiglu_packed,
                                      const void* w_out, void* out, const void* resid, long long rows, int c, int hidden,
                                      float eps, int dtype, void* stream) {
  KFB_CHECK_ARG(is_dtype(dtype), "transition_static: bad dtype %d", dtype);
  KFB_CHECK_ARG(rows >= 1 && c >= 8 && hidden >= 128, "transition_static: rows %lld c %d hidden %d", rows, c, hidden);
  // the fp32-accurate mode keeps six bf16 parts of every temporary: six times the bytes
  const size_t need = dtype == KFB_FP32_PRECISE ? kfb_transition_workspace_bytes_precise(rows, c, hidden)
                                                : kfb_transition_workspace_bytes(rows, c, hidden);
  if (need > kStaticScratchBytes) {
    set_error("transition_static: %lld rows x (c=%d + hidden=%d)%s need %zu bytes of scratch, the built-in array holds %zu; "
              "use kfb_transition_fwd with a caller-provided workspace for this size",
              rows, c, hidden, dtype == KFB_FP32_PRECISE ? " in the fp32-accurate mode" : "", need, kStaticScratchBytes);
    return KFB_ERR_UNSUPPORTED;
  }
  void* scratch = nullptr;
  KFB_TRY(static_scratch(&scratch));
  // Both temporaries are written in full (for the rows in use) before they are read, so nothing in
  // the array has to start at zero and stale contents of an earlier call are never observed.
  return kfb_transition_fwd(x, ln_w, ln_b, w_swiglu_packed, w_out, out, resid, scratch, kStaticScratchBytes, rows, c,
                            hidden, eps, dtype, stream);
}

}  // extern "C"
