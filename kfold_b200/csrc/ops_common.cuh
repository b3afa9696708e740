// Small helpers shared by the operator entry points.
#pragma once
#include "common.cuh"
#include "gemm.cuh"
#include "layernorm.cuh"

namespace kfb {

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
inline bool is_dtype(int d) { return d == KFB_BF16 || d == KFB_FP32 || d == KFB_FP32_PRECISE; }
inline bool is_fp32_io(int d) { return d == KFB_FP32 || d == KFB_FP32_PRECISE; }
inline size_t dtype_bytes(int d) { return d == KFB_BF16 ? 2 : 4; }

// Carves 256-byte aligned pieces out of a caller-provided workspace.
struct Carver {
  uint8_t* base;
  size_t off = 0;
  explicit Carver(void* p) : base(static_cast<uint8_t*>(p)) {}
  template <typename T>
  T* take(size_t count) {
    T* r = reinterpret_cast<T*>(base + off);
    off += align_up(count * sizeof(T), 256);
    return r;
  }
};

// Row-major output segment [rows][ld] starting at column 0.
inline EpiSeg row_major_seg(void* dst, int ncols, long long ld, long long s_o, long long s_b, int out_fp32, int col_begin = 0) {
  EpiSeg s = {};
  s.col_begin = col_begin;
  s.ncols = ncols;
  s.out_fp32 = out_fp32;
  s.dst = dst;
  s.s_col = 1;
  s.s_n = ld;
  s.s_o = s_o;
  s.s_b = s_b;
  const int v = out_fp32 ? 4 : 8;
  s.vec = (ld % v == 0) && (s_o % v == 0) && (s_b % v == 0) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
  return s;
}

}  // namespace kfb
