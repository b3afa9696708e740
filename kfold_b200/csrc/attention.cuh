// Flash-style attention with an additive pair bias and a key mask, on tcgen05/TMEM.
//
//   S = Q K^T + bias[h, q, k] + (mask[k] ? 0 : -1e9)        O = softmax_k(S) V   (optionally O *= sigmoid(G))
//
// Q arrives pre-scaled by log2(e)/sqrt(D): logits live in log2 units, the bias is multiplied by log2(e) as it is
// added.  One CTA handles 128 queries of one head for R (1 or 2) batch rows ("row groups") that share the same bias
// tile, walking the keys in half tiles of 64 with an online softmax; the L x L x H logits never exist in memory.
//   warp 0        TMA: K and V^T tiles per row group (3 stages), the 128 x 128 bias tile once for all R (2 stages)
//   warps 1..R    one MMA-issuing warp per row group, tcgen05.mma into tensor memory:
//                    S(t)  = Q K(t)^T + e0 maskrow(t)^T     (the key mask as a rank-1 K=16 step), triple-buffered
//                    O[c] += P_c(t) V_c(t)                   (A = P read from tensor memory), c = 0, 1
//   8 warps per row group = two softmax streams of four warps; stream c owns 32 of the 64 key columns of every half
//                 tile, one query row per thread: x = S + log2(e) bias (bias row from the swizzled shared-memory
//                 tile), P = exp2(x - s) against a lagging stabiliser s (the row maximum of the stream's first half
//                 tile, moved only when a half tile's row sum exceeds 2^100), P written as packed bf16 over the
//                 stream's own S columns.  Each stream has its own s, row sum and accumulator O[c] in tensor
//                 memory; the two are merged once at the end.
//
// Used for triangle attention (batch row = pair row i, bias shared by all rows, mask per row) and
// for pair-bias attention on the single / token track (bias shared by `bias_div` consecutive
// batch entries, mask per batch entry).
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"

namespace kfb {

struct AttnParams {
  int batch;      // independent attention problems (tri-att: B * N rows)
  int heads;
  int lq, lk;
  int d;          // real head dim (<= DPAD); output packs heads at stride d
  int dpad;       // padded head dim of q/k/v/g buffers: 32 or 64
  // q / k / g : position-major bf16, row index = batch * L + position, element stride ld*, head h at col0 + h*dpad
  const void* q; long long ldq; int q_col0;
  const void* k; long long ldk; int k_col0;
  // v^T : [batch][heads*dpad][ldv] bf16 (keys contiguous)
  const void* vt; long long ldv;
  // bias : [bias_batches][heads][lq][ldb] bf16 ; batch entry b uses bias batch b / bias_div, or, with bias_mod > 0,
  // (b / bias_div) * bias_mod + b % bias_mod: batch entries ordered (group, sample, window) with bias_mod windows and
  // bias_div = samples * windows, one bias per (group, window) that every sample of the group reuses
  const void* bias; long long ldb; int bias_div; int bias_mod;
  // 0: bias stored [bias_batches][heads][lq][ldb]; n > 0: stored [heads][n bias batches][lq][ldb] (head-major, as one
  // projection of all heads of several layers at once writes it)
  int bias_head_major;
  // window mode (atom transformers): batch entries are samples of lq == lk atoms; query q attends the 128 atoms
  // 32 (q / 32) - 48 ... + 79 (atoms outside [0, lk) count as masked), with one bias [32][128] per window:
  // bias_mod = lk / 32 windows per sample, bias_div = samples that share the biases.  A CTA takes 128 queries =
  // four windows and walks the 256 atoms that start 48 before them; a window's band inside that range is enforced
  // through the mask operand (one column per window), its bias rows are fetched by window-local key.
  int win;
  // key mask (0/1 bytes): element (b, k) at mask + b_hi*m_hi + b_lo*m_lo + k*m_k with b_hi = b / mask_lo_extent
  const unsigned char* mask; long long m_hi, m_lo, m_k; int mask_lo_extent;
  // optional gate logits, addressed like q
  const void* g; long long ldg; int g_col0;
  // output bf16: row (b, q) at out + (b*lq + q)*ldo, head h at column h*d
  void* out; long long ldo;
  long long* trace;  // debugging aid: when non-null, CTA (0,0,0) stores clock64() stamps of its pipeline events here
  const char* tag;  // name of the launch in the profile report (string literal), may be null
};

int launch_attention(cudaStream_t stream, const AttnParams& p);

// fp32-accurate mode: q, g and k, v are columns of fp32 row-major buffers (row = batch * L + position, `ld` / `ld_kv`
// floats per row, head h at col0 + h*d, no padding); bias fp32 [bias_batches][heads][lq][ldb]; the result is the
// bf16 triple split [rows][6 * heads * d].
struct AttnFp32Params {
  int batch, heads, lq, lk, d;
  const float *q, *k, *v, *g;  // same base pointer allowed; g may be null
  long long ld;                // row stride of q and g
  long long ld_kv;             // row stride of k and v (0: same as ld)
  int q_col0, k_col0, v_col0, g_col0;
  const float* bias; long long ldb; int bias_div; int bias_mod; int bias_head_major;  // as in AttnParams
  const unsigned char* mask; long long m_hi, m_lo, m_k; int mask_lo_extent;
  __nv_bfloat16* out6;
  const char* tag;
};
int launch_attention_fp32(cudaStream_t stream, const AttnFp32Params& p);

// Debugging aid: a device buffer of >= 512 long longs that receives pipeline time stamps (nullptr = off).
void set_attention_trace(long long* device_buffer);

}  // namespace kfb
