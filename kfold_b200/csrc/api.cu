// extern "C" entry points: argument checking and kernel sequencing.
#include "attention.cuh"
#include "ops_common.cuh"

using namespace kfb;

extern "C" {

KFB_API int kfb_version(void) { return 100; }

KFB_API const char* kfb_last_error(void) { return get_error(); }

KFB_API int kfb_device_status(int* code_out) {
  KFB_CUDA(cudaDeviceSynchronize());
  int code = 0, data_code = 0;
  const int zero = 0;
  KFB_CUDA(cudaMemcpyFromSymbol(&code, g_status, sizeof(int)));
  KFB_CUDA(cudaMemcpyFromSymbol(&data_code, g_data_status, sizeof(int)));
  if (code != 0) KFB_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(int)));
  if (data_code != 0) KFB_CUDA(cudaMemcpyToSymbol(g_data_status, &zero, sizeof(int)));
  if (code == 0) code = data_code;  // a wait that gave up outranks a data error
  if (code_out) *code_out = code;
  if (code != 0) {
    set_error("device-side error status %d (900: a token index out of range; otherwise a bounded wait that gave up)", code);
    return KFB_ERR_DEVICE_WAIT;
  }
  return KFB_OK;
}

KFB_API long long kfb_launch_count(void) { return launch_count(); }

#ifdef KFB_DEBUG_TRACE
// Development builds only (-DKFB_DEBUG_TRACE): a device buffer of at least 512 int64 receives clock stamps of the
// pipeline events of the first CTA of the attention kernel / of the GEMM launches whose profile tag equals `tag`.
KFB_API int kfb_debug_attention_trace(void* device_buffer_512_i64) {
  set_attention_trace(static_cast<long long*>(device_buffer_512_i64));
  return KFB_OK;
}

KFB_API int kfb_debug_gemm_trace(void* device_buffer_512_i64, const char* tag) {
  set_gemm_trace(static_cast<long long*>(device_buffer_512_i64), tag);
  return KFB_OK;
}
#endif

KFB_API int kfb_profile_enable(int on) {
  profile_enable(on != 0);
  return KFB_OK;
}

KFB_API int kfb_profile_report(char* buf, size_t cap) {
  KFB_CHECK_ARG(buf != nullptr && cap > 0, "profile_report: empty buffer");
  return profile_report(buf, cap) >= 0 ? KFB_OK : KFB_ERR_CUDA;
}

int kfb_layernorm(const void* x, void* y, const float* weight, const float* bias, long long rows, int c,
                  long long x_row_stride, long long y_row_stride, float eps, int in_dtype, int out_dtype, void* stream) {
  KFB_CHECK_ARG(x != nullptr && y != nullptr, "layernorm: null tensor");
  return launch_layernorm(as_stream(stream), x, y, weight, bias, rows, c, x_row_stride, y_row_stride, eps, in_dtype,
                          out_dtype);
}

KFB_API int kfb_layernorm_exchange(const void* x, void* y, const float* weight, const float* bias, int rows, int n, int c, float eps,
                                   int in_dtype, void* stream) {
  KFB_CHECK_ARG(x != nullptr && y != nullptr, "layernorm_exchange: null tensor");
  KFB_CHECK_ARG(rows >= 1 && n % rows == 0, "layernorm_exchange: N=%d must be a multiple of rows=%d", n, rows);
  RowPerm perm;
  perm.rows = rows;
  perm.n = n;
  return launch_layernorm(as_stream(stream), x, y, weight, bias, static_cast<long long>(rows) * n, c, c, c, eps, in_dtype, KFB_BF16,
                          perm);
}

KFB_API int kfb_gemm_bf16(const void* a, const void* b, void* d, const float* bias, int batch, int m, int n, int k, long long lda,
                  long long ldb, long long ldd, long long batch_stride_a, long long batch_stride_b,
                  long long batch_stride_d, int out_dtype, void* stream) {
  KFB_CHECK_ARG(a && b && d, "gemm: null tensor");
  KFB_CHECK_ARG(lda % 8 == 0 && ldb % 8 == 0, "gemm: lda/ldb must be multiples of 8 elements");
  GemmParams p = {};
  p.n_extent = m;
  p.o_extent = 1;
  p.batch = batch;
  p.n_cols = n;
  p.k_extent = k;
  p.b_batched = batch_stride_b != 0;
  p.nseg = 1;
  p.seg[0].col_begin = 0;
  p.seg[0].ncols = n;
  p.seg[0].out_fp32 = out_dtype == KFB_FP32;
  p.seg[0].dst = d;
  p.seg[0].s_col = 1;
  p.seg[0].s_n = ldd;
  p.seg[0].s_o = 0;
  p.seg[0].s_b = batch_stride_d;
  const int vec_elems = out_dtype == KFB_FP32 ? 4 : 8;
  p.seg[0].vec = (ldd % vec_elems == 0) && (batch_stride_d % vec_elems == 0) && ((reinterpret_cast<uintptr_t>(d) & 15) == 0);
  p.col_bias = bias;
  GemmOperandA oa = {a, lda, 0, batch_stride_a};
  GemmOperandB ob = {b, ldb, batch_stride_b};
  return launch_gemm_bf16(as_stream(stream), oa, ob, p);
}

}  // extern "C"
