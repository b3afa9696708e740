// Host-side helpers shared by the entry points: status codes, last-error text,
// and construction of TMA tensor maps through the driver entry point (the
// library links only against the CUDA runtime).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kfold_b200.h"

namespace kfb {

void set_error(const char* fmt, ...);
const char* get_error();

#define KFB_CHECK_ARG(cond, ...)        \
  do {                                  \
    if (!(cond)) {                      \
      ::kfb::set_error(__VA_ARGS__);    \
      return KFB_ERR_INVALID_ARGUMENT;  \
    }                                   \
  } while (0)

#define KFB_CUDA(expr)                                                                   \
  do {                                                                                   \
    cudaError_t e_ = (expr);                                                             \
    if (e_ != cudaSuccess) {                                                             \
      ::kfb::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, __LINE__); \
      return KFB_ERR_CUDA;                                                               \
    }                                                                                    \
  } while (0)

#define KFB_TRY(expr)            \
  do {                           \
    int s_ = (expr);             \
    if (s_ != KFB_OK) return s_; \
  } while (0)

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline int cdiv(int a, int b) { return (a + b - 1) / b; }

// Launch accounting.  Every kernel launch goes through a LaunchScope: it bumps the global launch
// counter and, while profiling is enabled, brackets the launch with CUDA events on its stream.
struct LaunchScope {
  LaunchScope(cudaStream_t stream, const char* tag);
  ~LaunchScope();
  cudaStream_t stream_;
  int slot_;
};

long long launch_count();
void profile_enable(bool on);
int profile_report(char* buf, size_t cap);

int sm_count();  // multiprocessors of the current device (cached per device)

// Encode a tiled tensor map.  dims/strides are given innermost first; strides[i] is the
// byte stride of dimension i+1 (dimension 0 is contiguous).  elem_bytes is 2 (bf16) or 4 (fp32).
// swizzle_bytes in {0, 32, 64, 128}: the inner box extent in bytes must equal it when non-zero.
int make_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, int swizzle_bytes);

}  // namespace kfb
