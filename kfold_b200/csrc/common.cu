// Status word, last-error text, device queries and TMA tensor-map encoding.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <algorithm>
#include <vector>

#include "common.cuh"
#include "ptx.cuh"

namespace kfb {

__device__ int g_status = 0;
__device__ int g_data_status = 0;

static thread_local char t_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
}
const char* get_error() { return t_error; }

// ------------------------------------------------------------------------------------------------
// launch counter + optional per-launch event timing
// ------------------------------------------------------------------------------------------------
namespace {
struct ProfRec {
  cudaEvent_t e0, e1;
  const char* tag;
};
std::mutex g_prof_mu;
std::vector<ProfRec> g_prof;
bool g_prof_on = false;
std::atomic<long long> g_launches{0};
}  // namespace

LaunchScope::LaunchScope(cudaStream_t stream, const char* tag) : stream_(stream), slot_(-1) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (!g_prof_on) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  ProfRec r;
  r.tag = tag;
  if (cudaEventCreate(&r.e0) != cudaSuccess || cudaEventCreate(&r.e1) != cudaSuccess) return;
  cudaEventRecord(r.e0, stream);
  g_prof.push_back(r);
  slot_ = static_cast<int>(g_prof.size()) - 1;
}
LaunchScope::~LaunchScope() {
  if (slot_ < 0) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (slot_ < static_cast<int>(g_prof.size())) cudaEventRecord(g_prof[slot_].e1, stream_);
}

long long launch_count() { return g_launches.load(); }

void profile_enable(bool on) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  for (auto& r : g_prof) {
    cudaEventDestroy(r.e0);
    cudaEventDestroy(r.e1);
  }
  g_prof.clear();
  g_prof_on = on;
}

// Writes one line per tag: "<tag> <launches> <total_ms> <large launches> <their total_ms>\n", "large" = the launches that
// took at least half as long as the tag's upper-quartile launch (a tag such as the transition's serves the pair tensor and the much
// smaller single track: the large group is the pair-sized work).  Synchronises on the recorded events.
int profile_report(char* buf, size_t cap) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  struct Agg { const char* tag; long long n; double ms; float mx; long long n_large; double ms_large; };
  std::vector<Agg> agg;
  std::vector<std::pair<int, float>> each;   // (index into agg, ms) per launch
  for (auto& r : g_prof) {
    if (cudaEventSynchronize(r.e1) != cudaSuccess) continue;
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, r.e0, r.e1) != cudaSuccess) continue;
    int idx = -1;
    for (size_t i = 0; i < agg.size(); ++i)
      if (strcmp(agg[i].tag, r.tag) == 0) { idx = static_cast<int>(i); break; }
    if (idx < 0) {
      agg.push_back({r.tag, 0, 0.0, 0.f, 0, 0.0});
      idx = static_cast<int>(agg.size()) - 1;
    }
    agg[idx].n++;
    agg[idx].ms += ms;
    if (ms > agg[idx].mx) agg[idx].mx = ms;
    each.emplace_back(idx, ms);
  }
  // the reference duration of a tag is its upper quartile, not its maximum: one launch that was held up (a clock change, a
  // neighbour on the GPU) must not make every other launch of the tag "small"
  for (size_t i = 0; i < agg.size(); ++i) {
    std::vector<float> v;
    for (auto& e : each)
      if (e.first == static_cast<int>(i)) v.push_back(e.second);
    std::sort(v.begin(), v.end());
    agg[i].mx = v.empty() ? 0.f : v[(v.size() * 3) / 4 < v.size() ? (v.size() * 3) / 4 : v.size() - 1];
  }
  for (auto& e : each)
    if (e.second >= 0.5f * agg[e.first].mx) { agg[e.first].n_large++; agg[e.first].ms_large += e.second; }
  size_t off = 0;
  for (auto& a : agg) {
    int w = snprintf(buf + off, off < cap ? cap - off : 0, "%s %lld %.6f %lld %.6f\n", a.tag, a.n, a.ms, a.n_large, a.ms_large);
    if (w < 0 || off + w >= cap) break;
    off += w;
  }
  if (cap) buf[off < cap ? off : cap - 1] = 0;
  return static_cast<int>(agg.size());
}

int sm_count() {
  static int cached[64];
  static std::once_flag once;
  std::call_once(once, [] { memset(cached, 0, sizeof(cached)); });
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, int swizzle_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return KFB_ERR_CUDA;
  }
  KFB_CHECK_ARG(rank >= 2 && rank <= 5, "tensor map rank %d out of range", rank);
  KFB_CHECK_ARG((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor map base %p is not 16-byte aligned", base);
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    KFB_CHECK_ARG(dims[i] >= 1 && box[i] >= 1 && box[i] <= 256, "tensor map dim %d: extent %llu box %u", i,
                  (unsigned long long)dims[i], box[i]);
  }
  for (int i = 0; i + 1 < rank; ++i) {
    uint64_t s = strides_bytes[i];
    if (dims[i + 1] == 1 && (s == 0 || (s & 15))) s = 16;  // never dereferenced beyond coordinate 0
    KFB_CHECK_ARG(s != 0 && (s & 15) == 0, "tensor map stride %d = %llu bytes is not a positive multiple of 16", i + 1,
                  (unsigned long long)s);
    gstr[i] = s;
  }
  CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
  if (swizzle_bytes == 128) sw = CU_TENSOR_MAP_SWIZZLE_128B;
  else if (swizzle_bytes == 64) sw = CU_TENSOR_MAP_SWIZZLE_64B;
  else if (swizzle_bytes == 32) sw = CU_TENSOR_MAP_SWIZZLE_32B;
  if (swizzle_bytes) KFB_CHECK_ARG((int)box[0] * elem_bytes == swizzle_bytes, "inner box %u x %d bytes != swizzle span %d",
                                   box[0], elem_bytes, swizzle_bytes);
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu %llu, box %u %u)", (int)r, rank,
              (unsigned long long)dims[0], (unsigned long long)dims[1], box[0], box[1]);
    return KFB_ERR_CUDA;
  }
  return KFB_OK;
}

}  // namespace kfb
