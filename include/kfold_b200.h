/*
 * kfold_b200 -- C ABI of the B200 (sm_100a) kernel backend for K-Fold's
 * Pairformer / diffusion hot path.
 *
 * The reference (SeonghwanSeo/kfold) has no native interface of its own: its
 * kernel backends are Python callables selected by a `kernel_backend` string
 * (src/kfold/utils/runtime.py:44-69) and invoked from the primitive modules.
 * Each entry point below therefore cites the reference *Python* call it stands
 * in for.  Conventions for every function:
 *
 *   - plain C, raw device pointers, explicit sizes, a `cudaStream_t` passed as
 *     `void*`; no torch types;
 *   - returns an `int` status (KFB_OK = 0); never throws, exits or synchronises
 *     the device (except kfb_device_status, which is a deliberate sync);
 *   - allocates nothing: every temporary lives in a caller-provided workspace
 *     whose size the matching `*_workspace_bytes` function reports;
 *   - launches on the stream passed in; safe to call from several host threads
 *     on different streams;
 *   - `dtype` is KFB_BF16 or KFB_FP32 and describes activations in and out;
 *     LayerNorm affine parameters are always fp32, projection weights are in
 *     the packed layouts produced by kfold_b200/packing.py.
 */
#ifndef KFOLD_B200_H_
#define KFOLD_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define KFB_API __attribute__((visibility("default")))
#else
#define KFB_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum {
  KFB_OK = 0,
  KFB_ERR_INVALID_ARGUMENT = 1,
  KFB_ERR_UNSUPPORTED = 2,
  KFB_ERR_CUDA = 3,
  KFB_ERR_DEVICE_WAIT = 4 /* a bounded device-side wait ran out; see kfb_device_status */
};

enum { KFB_BF16 = 0, KFB_FP32 = 1 };

/* Library version (major*10000 + minor*100 + patch). */
KFB_API int kfb_version(void);

/* Text of the last error raised on the calling host thread ("" if none). */
KFB_API const char* kfb_last_error(void);

/* Synchronises the current device and returns the device-side status word:
 * 0, or the code of the first bounded wait that gave up inside a kernel
 * (then also resets it).  For tests and post-mortems; not on the hot path. */
KFB_API int kfb_device_status(int* code_out);

/*
 * LayerNorm over the last dimension: y = (x - mean) * rstd * weight + bias, statistics in fp32.
 * Replaces LayerNorm.forward (src/kfold/model/primitives/normalization.py:61-91).
 * x, y: `rows` rows of `c` channels; row r starts at x + r*x_row_stride (elements).
 * weight / bias may be NULL (no scale / no offset, as AdaLN's inner norms use).
 */
KFB_API int kfb_layernorm(const void* x, void* y, const float* weight, const float* bias, long long rows, int c,
                  long long x_row_stride, long long y_row_stride, float eps, int in_dtype, int out_dtype, void* stream);

/*
 * Plain bf16 GEMM on the tcgen05 path: D[b, m, n] = sum_k A[b, m, k] * B[b, n, k]  (+ bias[n]).
 * The building block every projection and the triangle contraction run on; exported
 * so that it can be checked in isolation.  lda / ldb / ldd are row strides, the
 * batch strides may be 0 for B (shared weights).  out_dtype selects bf16 or fp32 D.
 */
KFB_API int kfb_gemm_bf16(const void* a, const void* b, void* d, const float* bias, int batch, int m, int n, int k, long long lda,
                  long long ldb, long long ldd, long long batch_stride_a, long long batch_stride_b,
                  long long batch_stride_d, int out_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KFOLD_B200_H_ */
