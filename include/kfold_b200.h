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

/* Activation dtype / arithmetic of an operator call:
 *   KFB_BF16          bf16 tensors, bf16 tensor-core arithmetic with fp32 accumulation;
 *   KFB_FP32          fp32 tensors in and out, same bf16 arithmetic inside (what autocast(bf16) on fp32 inputs gives);
 *   KFB_FP32_PRECISE  fp32 tensors and fp32-accurate arithmetic: every GEMM operand is split into three bf16 parts
 *                     (x = x0 + x1 + x2, 24 mantissa bits) and the six significant partial products are accumulated
 *                     in fp32 on the same tensor-core kernels; weights come from the `precise` packing.  Needs the
 *                     larger workspaces reported by the *_workspace_bytes_precise functions. */
enum { KFB_BF16 = 0, KFB_FP32 = 1, KFB_FP32_PRECISE = 2 };

/* Library version (major*10000 + minor*100 + patch). */
KFB_API int kfb_version(void);

/* Text of the last error raised on the calling host thread ("" if none). */
KFB_API const char* kfb_last_error(void);

/* Synchronises the current device and returns the device-side status:
 * 0, or the code of the first bounded wait that gave up inside a kernel, or
 * 900 when a kernel met a token index out of range (both are then reset).
 * Kernels never stop the process on such an error: a wait that gave up leaves
 * the tiles it was waiting for unwritten, and every later kernel on that device
 * abandons its waits early until the status is read.  Callers poll this at a
 * point where a device synchronisation is acceptable -- once per complex, or
 * once per sampler run -- and discard the results of that span when it is
 * non-zero.  A data error (900) does not affect other kernels. */
KFB_API int kfb_device_status(int* code_out);

/* Number of kernels this library has launched in the calling process so far. */
KFB_API long long kfb_launch_count(void);

/* Per-launch timing with CUDA events on the launch stream.  enable(1) clears old records and starts
 * recording, enable(0) stops.  report() waits for the recorded events and writes one text line per
 * launch tag: "<tag> <launches> <total_ms> <large launches> <their total_ms>\n", "large" = the launches that took at
 * least half as long as the tag's upper-quartile launch (the pair-sized ones of a tag that also serves the single track).
 * Creates events while enabled; off by default. */
KFB_API int kfb_profile_enable(int on);
KFB_API int kfb_profile_report(char* buf, size_t cap);

/*
 * Triangle multiplicative update, outgoing (incoming = 0) or incoming (incoming = 1).
 * Replaces TriangleMultiplicationOutgoing.forward / TriangleMultiplicationIncoming.forward
 * (src/kfold/model/primitives/triangle_multiplication.py:179-229 and :263-313) and the Triton
 * entry point `forward(x, cached, direction, mask, eps)` called at :138-144.
 *   x, out : (batch, n, n, c) contiguous, `dtype`; n a multiple of 8, c a multiple of 64.
 *   mask   : (batch, n, n) bytes, non-zero = valid.
 *   w_in_packed : bf16 [4c, c], linear_p_in / linear_g_in interleaved in blocks of 128 rows
 *                 (value rows of 128 channels, then their gate rows), BOTH multiplied by 0.5 (exact in bf16): the
 *                 epilogue evaluates v sigmoid(g) as v' + v' tanh(g') with v' = v / 2, g' = g / 2.  With
 *                 KFB_FP32_PRECISE the matrices are unscaled (bf16 triple splits, exact sigmoid).
 *   w_gout, w_pout : bf16 [c, c] (linear_g_out, linear_p_out);  ln_* : fp32 [c].
 *   resid  : NULL, or a (batch, n, n, c) tensor of `dtype` added to the update (may equal x and out).
 * Writes out = update (+ resid).  Arithmetic: bf16 operands, fp32 accumulation and statistics.
 */
KFB_API size_t kfb_trimul_workspace_bytes(int batch, int n, int c);
KFB_API size_t kfb_trimul_workspace_bytes_precise(int batch, int n, int c);
KFB_API int kfb_trimul_fwd(int incoming, const void* x, const unsigned char* mask, const float* ln_in_w,
                           const float* ln_in_b, const void* w_in_packed, const void* w_gout, const float* ln_out_w,
                           const float* ln_out_b, const void* w_pout, void* out, const void* resid, void* workspace,
                           size_t workspace_bytes, int batch, int n, int c, float eps, int dtype, void* stream);

/*
 * Triangle attention around the starting node (ending = 0) or the ending node (ending = 1).
 * Replaces TriangleAttention.forward + MultiHeadAttention.forward
 * (src/kfold/model/primitives/triangle_attention.py:375-434, :285-335) and the Triton entry
 * `triton_triangular_attn(module, x, mask)` (:63-129).  The ending node is handled inside: pass
 * the untransposed x and mask.
 *   x, out : (batch, n, n, c) contiguous, `dtype`;  mask : (batch, n, n) bytes.
 *   w_proj_packed : bf16 [4*heads*dp + 32, c] = [Wq/sqrt(d) | Wk | Wg | Wv | Wz], every head padded
 *                   from d = c/heads to dp (32 if d <= 32 else 64) rows, Wz padded to 32 rows.
 *   w_out  : bf16 [c, c] (mha.linear_o);  resid as for kfb_trimul_fwd.
 * Masked keys get an additive -1e9 (the reference's `inf`), so a fully masked row yields the
 * uniform average of V, exactly as the reference does.  batch*n must not exceed 65535.
 */
KFB_API size_t kfb_triatt_workspace_bytes(int batch, int n, int c, int heads);
KFB_API size_t kfb_triatt_workspace_bytes_precise(int batch, int n, int c, int heads);
KFB_API int kfb_triatt_fwd(int ending, const void* x, const unsigned char* mask, const float* ln_w, const float* ln_b,
                           const void* w_proj_packed, const void* w_out, void* out, const void* resid, void* workspace,
                           size_t workspace_bytes, int batch, int n, int c, int heads, float eps, int dtype, void* stream);

/*
 * Row-sharded forms (no counterpart in the reference, which never splits a pair tensor across GPUs; they are
 * the two halves of the functions above, cut where the collective goes).  A rank holds `rows` of the n pair
 * rows as x (rows, n, c).
 *   kfb_trimul_project : LayerNorm + gated input projection (if w_in_packed) -> ab_out bf16 [2c][rows][n]
 *                        (operand a = first c channels, b = last c), + output-gate logits (if w_gout)
 *                        -> gl_out bf16 [rows*n][c].  xn_scratch: bf16 [rows*n][c].  x == NULL: xn_scratch already holds
 *                        the normalised rows (a second call on the same tensor, e.g. the gate logits issued after the
 *                        operands so that they run under the operands' exchange).  transposed != 0: the operands are
 *                        written transposed, ab_out [2c][n][rows] (the incoming direction's a[k][i] at [i][k]).
 *                        parts > 1 (4c a multiple of 256 * parts): only part `part` of the 2c operand channels, in the
 *                        packed order, into ab_out = that part's buffer [2c / parts][..][..] -- the caller starts the
 *                        exchange of one part while the next is projected.
 *   kfb_trimul_contract : the contraction alone on `cpart` channels (a, t: [cpart][rows][n]; b in gathered pieces), so that
 *                        one half of the channels is contracted while the other half's operand is still in flight.
 *   (the caller all-gathers operand b: every rank's [c][rows][n] piece, rank after rank)
 *   kfb_trimul_finish  : contraction of the local a rows against all rows of b, LayerNorm_out, gated output
 *                        projection (+ resid).  b_gathered: pieces of b_piece_rows rows, b_piece_stride elements
 *                        apart.  t_scratch / tn_scratch: bf16 [c*rows*n] each.  out/resid: (rows, n, c).
 * The incoming direction is the same pair of calls with ab taken from the TRANSPOSED shard (the caller
 * transposes z across ranks with an all-to-all) and gl / resid from the row shard -- or, with the channel-sharded
 * exchange below, the transposed projection of the row shard itself and no transpose of z.
 *   kfb_triatt_project : LayerNorm + projection -> qkg_out bf16 [rows*n][3*heads*dp], vt_out bf16
 *                        [rows][heads*dp][n], bias_out bf16 [heads][rows][n] (the caller all-gathers it per head
 *                        into [heads][n][n]).
 *   kfb_triatt_finish  : attention of the local rows against the full bias, output projection (+ resid).
 *                        mask: (rows, n) bytes; og_scratch: bf16 [rows*n][c].
 * Ending node without reorder copies (exchange_layout != 0; rows must divide n):
 *   kfb_layernorm_exchange : LayerNorm of the row shard x (rows, n, c), written bf16 as the send buffer of the shard
 *                        transpose, [q][i][j][c] = LN(x[i][q*rows + j]) -- block q goes to rank q.
 *   kfb_triatt_project with exchange_layout: x = the received buffer [q][i_q][j][c] (already normalised, bf16; ln_w, ln_b,
 *                        xn_scratch unused); outputs as above for the transposed shard (row j, position q*rows + i_q).
 *   kfb_triatt_finish with exchange_layout: out = the update as the send buffer of the transpose back,
 *                        bf16 [q][j][k_q][c] for position (j, q*rows + k_q); no residual.
 *   kfb_pair_bias_rows_fwd : kfb_pair_bias_fwd on a shard: z (rows, n, c) -> bf16 [heads][rows][n].
 */
KFB_API int kfb_trimul_project(const void* x, const unsigned char* mask, const float* ln_in_w, const float* ln_in_b,
                               const void* w_in_packed, const void* w_gout, void* xn_scratch, void* ab_out, void* gl_out,
                               int batch, int rows, int n, int c, int transposed, int part, int parts, float eps, int dtype,
                               void* stream);
KFB_API int kfb_trimul_contract(const void* a, const void* b_gathered, int b_piece_rows, long long b_piece_stride, void* t, int rows,
                                int n, int cpart, void* stream);
KFB_API int kfb_trimul_finish(const void* a, const void* b_gathered, int b_piece_rows, long long b_piece_stride,
                              const void* gl, const float* ln_out_w, const float* ln_out_b, const void* w_pout,
                              void* t_scratch, void* tn_scratch, void* out, const void* resid, int rows, int n, int c,
                              float eps, int dtype, void* stream);
/* Channel-sharded contraction for the row-sharded pair track (the cheaper exchange: an all-to-all of a and b to a
 * channel-sharded layout, this call, an all-to-all of t back; kfb_trimul_finish is then called with a = b = NULL and
 * t_scratch = the received t).  ab_recv: bf16 [world][2][cl][rows][n] as received; t_send: bf16 [world][cl][rows][n].
 * incoming != 0: the ranks projected with transposed != 0, ab_recv is [world][2][cl][n][rows], and the product is
 * t[i][j] = sum_k a[k][i] b[k][j] with K in `world` pieces (rows a multiple of 64). */
KFB_API int kfb_trimul_contract_cs(const void* ab_recv, void* t_send, int world, int rows, int n, int cl, int incoming, void* stream);
KFB_API int kfb_triatt_project(const void* x, const float* ln_w, const float* ln_b, const void* w_proj_packed,
                               void* xn_scratch, void* qkg_out, void* vt_out, void* bias_out, int rows, int n, int c,
                               int heads, int exchange_layout, float eps, int dtype, void* stream);
KFB_API int kfb_layernorm_exchange(const void* x, void* y, const float* weight, const float* bias, int rows, int n, int c, float eps,
                                   int in_dtype, void* stream);
KFB_API int kfb_pair_bias_rows_fwd(const void* z, const float* ln_w, const float* ln_b, const void* w, void* bias_out,
                                   void* workspace, size_t workspace_bytes, int rows, int n, int c, int heads, float eps,
                                   int dtype, void* stream);
KFB_API int kfb_triatt_finish(const void* qkg, const void* vt, const void* bias_full, const unsigned char* mask,
                              const void* w_out, void* og_scratch, void* out, const void* resid, int rows, int n, int c,
                              int heads, int exchange_layout, int dtype, void* stream);

/*
 * bias[b, h, i, j] = sum_c LayerNorm(z)[b, i, j, c] * w[h, c], written bf16 as (batch, heads, n, n).
 * Replaces `linear_pair_bias(layernorm_z(z)).movedim(-1, -3)`
 * (src/kfold/model/modules/confidence_head.py:162-163) and DiffusionStack.get_pair_bias
 * (src/kfold/model/layers/folding/diffusion.py:411-416).  w : bf16 [heads, c].
 * With transposed != 0 the result is written as bias_out[b, h, j, i].
 */
KFB_API size_t kfb_pair_bias_workspace_bytes(int batch, int n, int c);
KFB_API size_t kfb_pair_bias_workspace_bytes_precise(int batch, int n, int c);
KFB_API int kfb_pair_bias_fwd(const void* z, const float* ln_w, const float* ln_b, const void* w, void* bias_out,
                              void* workspace, size_t workspace_bytes, int batch, int n, int c, int heads, int transposed,
                              float eps, int dtype, void* stream);

/*
 * Gated self-attention with pair bias on already-normalised input.
 * Replaces `attention_pair_bias(module, x_q, x_k, pair_bias, mask, kernel_backend=..., call_site=...)`
 * with x_q is x_k (src/kfold/model/primitives/attention.py:28-94; torch kernel :239-271).
 *   x : bf16 (batch, l, c);  pair_bias : bf16 (batch / bias_div, heads, l, l) -- `bias_div` consecutive
 *   batch entries share one bias (the diffusion samples);  mask : (batch, l) bytes;  l multiple of 8.
 *   w_proj_packed : bf16 [4*heads*dp, c] = [Wq/sqrt(d) | Wk | Wg | Wv], heads padded to dp;
 *   proj_bias : fp32 [4*heads*dp] (scaled q bias in the first quarter) or NULL;
 *   w_out : bf16 [c, c];  out_bias : fp32 [c] or NULL;  out : (batch, l, c) of `out_dtype`;
 *   out_gate : NULL, or bf16 logits (batch / gate_share, l, c): out *= sigmoid(out_gate) -- the AdaLN-Zero output
 *   gate sigmoid(Linear(s)) of SelfAttentionPairBias.forward (src/kfold/model/layers/folding/
 *   attention_pair_bias.py:155-157), shared by `gate_share` consecutive batch entries;
 *   resid : NULL or a tensor like out that is added.
 * With out_dtype = KFB_FP32_PRECISE every tensor argument (x, pair_bias, out_gate, out, resid) is fp32, the weights
 * come from the precise packing (heads not padded) and the attention core runs on the fp32 CUDA-core kernel.
 */
KFB_API size_t kfb_apb_workspace_bytes(int batch, int l, int c, int heads);
KFB_API size_t kfb_apb_workspace_bytes_precise(int batch, int l, int c);
KFB_API int kfb_apb_fwd(const void* x, const void* pair_bias, const unsigned char* mask, const void* w_proj_packed,
                        const float* proj_bias, const void* w_out, const float* out_bias, const void* out_gate,
                        int gate_share, long long gate_ld, void* out, const void* resid, void* workspace,
                        size_t workspace_bytes, int batch, int l, int c, int heads, int bias_div, int out_dtype, void* stream);

/*
 * Gated cross attention with pair bias on already-normalised inputs: queries from x_q, keys and values from x_k.
 * Replaces `attention_pair_bias(module, x_q, x_k, pair_bias, mask, kernel_backend=..., call_site="diffusion_local")`
 * (src/kfold/model/primitives/attention.py:28-94; torch kernel :239-271) as CrossAttentionPairBias.forward calls it
 * on the atom windows (src/kfold/model/layers/folding/attention_pair_bias.py:206-260; windows of 32 queries and
 * 128 keys built by src/kfold/model/layers/folding/utils.py:97-188).
 *   x_q : bf16 (batch, lq, c);  x_k : bf16 (batch, lk, c);  mask : (batch, lk) bytes;  lq, lk multiples of 8.
 *   pair_bias : bf16 (bias batches, heads, lq, lk).  Batch entry b uses bias batch b / bias_div when bias_mod == 0;
 *   with bias_mod > 0 the batch is ordered (group, sample, window), bias_mod = windows, bias_div = samples * windows,
 *   and entry b uses bias batch (b / bias_div) * bias_mod + b % bias_mod: one bias per (group, window), shared by the
 *   diffusion samples.  bias_head_major = 0: stored as above; n > 0: stored (heads, n bias batches, lq, lk), the layout
 *   kfb_window_bias_fwd writes.
 *   w_q_packed : bf16 [2*heads*dp, c] = [Wq * log2(e)/sqrt(d) | Wg], heads padded to dp;  q_bias : fp32 [2*heads*dp]
 *   (scaled q bias, gate bias) or NULL;  w_kv_packed : bf16 [2*heads*dp, c] = [Wk | Wv];
 *   w_out : bf16 [c, c];  out_bias : fp32 [c] or NULL;  out : (batch, lq, c) of `out_dtype`;
 *   out_gate : NULL, or bf16 logits (gate_rows, c): row r of the batch * lq query rows is multiplied by
 *   sigmoid(out_gate[r % gate_rows]) -- the output gate sigmoid(Linear(s_q)) of CrossAttentionPairBias.forward
 *   (:258-259), stored once when the samples share their conditioning;  resid : NULL or a tensor like out that is added.
 * With out_dtype = KFB_FP32_PRECISE every tensor argument is fp32, the weights are bf16 triple splits with unpadded
 * heads ([2c, 6c] each) and the attention core runs on the fp32 CUDA-core kernel.
 */
KFB_API size_t kfb_apb_cross_workspace_bytes(int batch, int lq, int lk, int c, int heads);
KFB_API size_t kfb_apb_cross_workspace_bytes_precise(int batch, int lq, int lk, int c);
KFB_API int kfb_apb_cross_fwd(const void* x_q, const void* x_k, const void* pair_bias, const unsigned char* mask,
                              const void* w_q_packed, const float* q_bias, const void* w_kv_packed, const void* w_out,
                              const float* out_bias, const void* out_gate, long long gate_rows, long long gate_ld, void* out,
                              const void* resid, void* workspace, size_t workspace_bytes, int batch, int lq, int lk, int c, int heads,
                              int bias_div, int bias_mod, int bias_head_major, int out_dtype, void* stream);

/*
 * The same attention on the UN-windowed atoms (bf16 compute, head dim <= 32): the windows of 32 queries and 128 keys
 * (atoms 32 w - 48 ... 32 w + 79 for window w, src/kfold/model/layers/folding/utils.py:97-188) are walked by the
 * kernel itself, so neither queries, keys nor conditionings are gathered and the key / value projection runs once
 * per atom instead of once per window slot.
 *   x_q, x_k : bf16 (batch, l, c), the query-side and key-side normalised atoms, l a multiple of 32;
 *   pair_bias : bf16, one [32][128] bias per window and head: (bias groups * l/32, heads, 32, 128), or head-major
 *   (heads, n, 32, 128) with bias_head_major = n >= bias groups * l/32;  `bias_share` consecutive batch entries
 *   (samples) use the same biases;  mask : bytes (batch / mask_share, l), atom validity;
 *   weights, out_gate / gate_rows, out, resid as in kfb_apb_cross_fwd; out_dtype KFB_BF16 or KFB_FP32 (output only).
 */
KFB_API size_t kfb_apb_window_workspace_bytes(int batch, int l, int c, int heads);
KFB_API int kfb_apb_window_fwd(const void* x_q, const void* x_k, const void* pair_bias, const unsigned char* mask,
                               const void* w_q_packed, const float* q_bias, const void* w_kv_packed, const void* w_out,
                               const float* out_bias, const void* out_gate, long long gate_rows, long long gate_ld, void* out,
                               const void* resid, void* workspace, size_t workspace_bytes, int batch, int l, int c, int heads, int bias_share,
                               int mask_share, int bias_head_major, int out_dtype, void* stream);

/*
 * Pair bias of the atom windows for every block of a local transformer at once:
 * bias[h, p] = sum_k LayerNorm(z[p])[k] * w[h, k].  Replaces `self.layernorm_z(z)` of LocalTransformerStack.forward
 * (src/kfold/model/layers/folding/diffusion_transformer.py:496) and the `linear_z_to_bias` of each block (:590-591)
 * with their weights stacked into w [heads = blocks * H, c].
 *   z : (positions, c) with positions = windows * 32 * 128, c in {16, 32, 64};  ln_w / ln_b : fp32 [c] or NULL;
 *   bias_out : (heads, positions), head-major (the `bias_head_major` layout of kfb_apb_cross_fwd).
 *   dtype KFB_BF16: z, w, bias_out bf16 (the normalised value is rounded to bf16 before the projection, fp32
 *   accumulation); KFB_FP32 or KFB_FP32_PRECISE: all three fp32.  normalise == 0 skips the LayerNorm (z already
 *   normalised: the per-block form of LocalTransformerBlock.forward).
 */
KFB_API int kfb_window_bias_fwd(const void* z, const float* ln_w, const float* ln_b, const void* w, void* bias_out,
                                long long positions, int c, int heads, float eps, int normalise, int dtype, void* stream);

/*
 * Token <-> atom maps and the small projections of the atom attention encoder / decoder
 * (src/kfold/model/layers/folding/atom_transformer.py:263-389 and :392-489).
 *   kfb_tokens_to_atoms replaces broadcast_tokens_to_atoms (src/kfold/model/layers/folding/utils.py:25-51) and the skip
 *     connection behind it (atom_transformer.py:468-470): out[b, a, :] = x[b, token_index[b / index_div, a], :]
 *     (+ addend[b, a, :]);  x (batch, n_token, d) of x_dtype, addend (NULL or like out) and out (batch, n_atom, d) of
 *     out_dtype (bf16 -> bf16, bf16 -> fp32, fp32 -> fp32).  An index outside [0, n_token) gives a zero row and sets
 *     the device status word (kfb_device_status) to 900.
 *   kfb_atoms_to_tokens replaces aggregate_atoms_to_tokens (utils.py:54-93): out[b, t, :] = mean of x[b, a, :] over the
 *     atoms with mask[a] != 0 and token_index[a] == t, accumulated in fp32 in atom order; a token without atoms gives
 *     zeros;  `relu` != 0 applies max(., 0) to x first (the ReLU of atom_transformer.py:384).
 *     x (batch, n_atom, d), out (batch, n_token, d), both of `dtype`.  workspace: NULL (every token scans all atoms) or
 *     kfb_atoms_to_tokens_workspace_bytes bytes, in which two small kernels first record each token's first and last
 *     atom so that the mean scans only that range (same result, any atom order).
 *   token_index : int64 (batch / index_div, n_atom), mask : bytes of the same shape -- `index_div` consecutive batch
 *   entries (the diffusion samples) share one row.
 *   kfb_coord_embed replaces `q + linear_r_to_q(r_noisy)` (atom_transformer.py:362-367, a float32 Linear):
 *     out[row, :] = q[qrow, :] + w r[row, :];  q (rows / samples, c) of q_dtype shared by the `samples` samples
 *     (rows ordered (group, sample, l atoms)), r fp32 (rows, kc <= 8: the sampler passes the scaled noisy
 *     coordinates and the scaled prior coordinates side by side, kc = 6), w fp32 [c, kc], out fp32 (rows, c);
 *     mask : NULL or bytes (rows / samples), atom validity shared like q: the coordinates of padding atoms count as zero
 *     (`r_noisy * atom_mask`, src/kfold/model/layers/folding/diffusion.py:521).
 *   kfb_ln_project replaces `linear_q_to_r(layernorm_q(q.float()))` (atom_transformer.py:487-488):
 *     out[row, j] = sum_i LayerNorm(x[row])[i] w[j, i];  x (rows, c) of dtype, ln_w / ln_b fp32 [c] or NULL,
 *     w fp32 [n_out <= 8, c], out fp32 (rows, n_out);  mask : NULL or bytes (rows / samples) with rows ordered
 *     (group, sample, l atoms): rows of padding atoms give zeros (`r_update * atom_mask`, diffusion.py:596).
 */
KFB_API int kfb_tokens_to_atoms(const void* x, const long long* token_index, const void* addend, void* out, int batch,
                                int n_token, int n_atom, int d, int index_div, int x_dtype, int out_dtype, void* stream);
KFB_API size_t kfb_atoms_to_tokens_workspace_bytes(int batch, int n_token, int index_div);
KFB_API int kfb_atoms_to_tokens(const void* x, const long long* token_index, const unsigned char* mask, void* out, void* workspace,
                                size_t workspace_bytes, int batch, int n_atom, int n_token, int d, int index_div, int relu,
                                int dtype, void* stream);
KFB_API int kfb_coord_embed(const void* q, const float* r, const float* w, const unsigned char* mask, float* out, long long rows,
                            int c, int kc, int samples, int l, int q_dtype, void* stream);
KFB_API int kfb_ln_project(const void* x, const float* ln_w, const float* ln_b, const float* w, const unsigned char* mask,
                           float* out, long long rows, int c, int n_out, float eps, int samples, int l, int dtype, void* stream);

/*
 * Adaptive LayerNorm: out = sigmoid(g) * LayerNorm(a) + v, LayerNorm without affine (fp32 statistics).
 * Replaces the last line of AdaLN.forward (src/kfold/model/primitives/normalization.py:117-125); the two
 * small projections of the conditioning, g = Linear(LN_s(s)) and v = LinearNoBias(LN_s(s)), are computed by
 * the caller (kfb_layernorm + kfb_gemm_bf16) once per token and passed as `gate_shift`: bf16 [rows / samples, 2c]
 * (logits g, then v).  a : (rows, c) of `in_dtype`, rows ordered (group, sample, position) with `l` positions;
 * the `samples` diffusion samples of a group share one conditioning row per position.  out : bf16 (rows, c).
 * gate_shift_ld (here) and gate_ld (kfb_apb_fwd, kfb_apb_cross_fwd, kfb_apb_window_fwd, kfb_cond_transition_fwd) are the
 * element strides between consecutive rows of those tables, 0 for densely packed rows: the conditioning projections of
 * all blocks of a stack can then be computed by one GEMM into one wide table of which every block reads its columns.
 */
KFB_API int kfb_adaln_fwd(const void* a, const void* gate_shift, long long gate_shift_ld, void* out, long long rows, int c,
                          int samples, int l, float eps, int in_dtype, void* stream);

/*
 * Conditioned transition: out = sigmoid(gate) * Linear_out(silu(u_a) * u_b) (+ resid), [u_a, u_b] = Linear(x).
 * Replaces lines 2-3 of ConditionedTransitionBlock.forward
 * (src/kfold/model/layers/folding/diffusion_transformer.py:73-81); x is the AdaLN output (kfb_adaln_fwd),
 * out_gate : bf16 logits [rows / samples, c] = Linear(s) + bias, shared by the samples of a group.
 */
KFB_API size_t kfb_cond_transition_workspace_bytes(long long rows, int hidden);
KFB_API size_t kfb_cond_transition_workspace_bytes_precise(long long rows, int c, int hidden);

/* y = x W^T (+ bias) at fp32 accuracy on the tensor core: x fp32 [rows, k], w6 = the bf16 triple split of W
 * [n, 6k] (kfold_b200.packing.split3_weights), bias fp32 [n] or NULL, out fp32 [rows, n].  The small projections of
 * the conditioning in the float32 sampler (src/kfold/model/primitives/normalization.py:117-125,
 * src/kfold/model/layers/folding/attention_pair_bias.py:151-156). */
KFB_API size_t kfb_linear_fp32_workspace_bytes(long long rows, int k);
KFB_API int kfb_linear_fp32(const void* x, const void* w6, const float* bias, void* out, void* workspace,
                            size_t workspace_bytes, long long rows, int n, int k, void* stream);
/* out = LayerNorm(x) W^T (+ bias) (+ resid) at fp32 accuracy (kfb_linear_fp32 with the LayerNorm and the residual fused):
 * `a + linear_s_to_a(layernorm_s(s))` of DiffusionStack.step (src/kfold/model/layers/folding/diffusion.py:568).
 * x, resid, out fp32; ln_w / ln_b fp32 [k] or NULL; normalise == 0 skips the LayerNorm; workspace as kfb_linear_fp32. */
KFB_API int kfb_ln_linear_fp32(const void* x, const float* ln_w, const float* ln_b, const void* w6, const float* bias,
                               const void* resid, void* out, void* workspace, size_t workspace_bytes, long long rows, int n, int k,
                               float eps, int normalise, void* stream);
KFB_API int kfb_cond_transition_fwd(const void* x_normed, const void* w_swiglu_packed, const void* w_out,
                                    const void* out_gate, long long gate_ld, void* out, const void* resid, void* workspace,
                                    size_t workspace_bytes, long long rows, int c, int hidden, int samples, int l, int dtype,
                                    void* stream);

/*
 * Pieces of SingleConditioning.forward (src/kfold/model/layers/folding/diffusion.py:122-152), all fp32:
 *   kfb_fourier_embed replaces FourierEmbedding.forward (src/kfold/model/layers/folding/embeddings.py:159-174):
 *     out[row, j] = cos(2 pi t[row] w[j] + b[j]);  t [rows], w and b [dim], out (rows, dim).
 *   kfb_broadcast_add replaces `s[:, None, :, :] + fourier_embed[:, :, None, :]` (diffusion.py:146):
 *     out[g, n, l, :] = s[g, l, :] + f[g, n, :];  s (groups, l, c), f (groups, samples, c), out (groups, samples, l, c).
 */
KFB_API int kfb_fourier_embed(const float* t, const float* w, const float* b, float* out, int rows, int dim, void* stream);
KFB_API int kfb_broadcast_add(const float* s, const float* f, float* out, int groups, int samples, int l, int c, void* stream);

/*
 * Callers of the pair stacks in the trunk (src/kfold/model/model.py:477-534).
 *   kfb_parcae_fwd replaces the recurrence between recycling iterations, `z = a * z + F.linear(self.layernorm_z(u_t), b)`
 *     (model.py:528): out = a (per channel) * z + LayerNorm(u) b^T.  z, u, out : (rows, c) of `dtype` (KFB_BF16 or KFB_FP32;
 *     bf16 arithmetic, fp32 accumulation -- the reference casts a and b to the autocast dtype, model.py:505);
 *     a : fp32 [c];  b_w : bf16 [c, c];  ln_w / ln_b : fp32 [c] or NULL.  out may equal z.
 *   kfb_lm_pair_features replaces `torch.cat([xi * xj, xi - xj], dim=-1)` of LMToPair.forward (model.py:128-131):
 *     x (batch, n, 2 d) of `dtype` = [xi | xj] per token -> out bf16 (batch, n, n, 2 d).
 *   kfb_gelu replaces torch.nn.GELU() (erf form) inside LMToPair's MLP (model.py:120-124), element-wise.
 */
KFB_API size_t kfb_parcae_workspace_bytes(long long rows, int c);
KFB_API int kfb_parcae_fwd(const void* z, const void* u, const float* ln_w, const float* ln_b, const float* a, const void* b_w,
                           void* out, void* workspace, size_t workspace_bytes, long long rows, int c, float eps, int dtype,
                           void* stream);
KFB_API int kfb_lm_pair_features(const void* x, void* out, int batch, int n, int d, int dtype, void* stream);
KFB_API int kfb_gelu(const void* x, void* y, long long n, int in_dtype, int out_dtype, void* stream);

/*
 * Pair conditioning of the diffusion module (src/kfold/model/layers/folding/diffusion.py:84-90): replaces
 * `self.layernorm(torch.cat([z, rel_pos_feats], dim=-1))` in one pass.  z (rows, c1) of z_dtype, rel (rows, c2) of rel_dtype
 * (KFB_BF16 or KFB_FP32 each) -> out fp32 (rows, k_pad): LayerNorm over the c1 + c2 concatenated channels (ln_w / ln_b fp32
 * [c1 + c2] or NULL), columns c1 + c2 .. k_pad - 1 zero so that the row feeds kfb_linear_fp32 (K a multiple of 8).
 * k_pad <= 512.
 */
KFB_API int kfb_concat_layernorm(const void* z, int z_dtype, const void* rel, int rel_dtype, const float* ln_w, const float* ln_b,
                                 float* out, long long rows, int c1, int c2, int k_pad, float eps, void* stream);
/*
 * The same with the relative-position encoding computed inside the kernel instead of read: replaces
 * `self.rel_pos_encoding(f_input, z.dtype)` (src/kfold/model/layers/folding/embeddings.py:58-130, AF3 Algorithm 3) together with
 * the concatenation and the LayerNorm; the (batch, n, n, 4 (r_max + 1) + 2 (s_max + 1) + 1) one-hot tensor never exists.
 * asym_id, residue_index, entity_id, token_index, sym_id: int64 [batch][n] (the fields of FoldingInput.token).  z (batch, n, n, c1).
 */
KFB_API int kfb_relpos_concat_layernorm(const void* z, int z_dtype, const long long* asym_id, const long long* residue_index,
                                        const long long* entity_id, const long long* token_index, const long long* sym_id,
                                        int r_max, int s_max, const float* ln_w, const float* ln_b, float* out, int batch, int n, int c1,
                                        int k_pad, float eps, void* stream);

/*
 * Pair-tensor preparation of the confidence head (src/kfold/model/modules/confidence_head.py:306-470).
 *   kfb_pair_outer_add replaces `z + self.linear_s1(s_inputs)[..., None, :, :] + self.linear_s2(s_inputs)[..., :, None, :]`
 *     (:347-351): out[b, i, j, :] = z[b, i, j, :] + row_add[b, j, :] + col_add[b, i, :];  z, out (batch, n, n, c), row_add and
 *     col_add (batch, n, c), all of `dtype`; c a multiple of 4.
 *   kfb_distogram_embed_add replaces the distogram embedding of forward_single (:449-455): out = z + w_t[bin(|x_i - x_j|)],
 *     bin = the number of `boundaries` (fp32, ascending) below the distance;  x fp32 (batch, n, 3), w_t (n_boundaries + 1, c)
 *     = linear_distogram.weight transposed, of `dtype` like z and out.
 */
KFB_API int kfb_pair_outer_add(const void* z, const void* row_add, const void* col_add, void* out, int batch, int n, int c, int dtype,
                               void* stream);
KFB_API int kfb_distogram_embed_add(const void* z, const float* x, const float* boundaries, int n_boundaries, const void* w_t, void* out,
                                    int batch, int n, int c, int dtype, void* stream);

/*
 * The coordinate-space steps of the sampler loop around the score network, KFoldECSI.sample_structure
 * (src/kfold/model/modules/ecsi.py:498-560).  A coordinate set is one diffusion sample of one complex: l atoms x 3 fp32,
 * contiguous; the n sets of a call are ordered (complex, sample) and `mask_div` consecutive sets share one row of the
 * atom mask (bytes, (n / mask_div, l)).  The host keeps the scalar schedule (times, bridge coefficients, churn and update
 * coefficients) and draws the normals -- in the reference's order, so that a run with the same generator state consumes
 * the same numbers -- and passes them in.
 *   kfb_coords_augment replaces CenterRandomAugmentation with centering=False (src/kfold/utils/geometry/random_augment.py:
 *     463-513): x <- x R + trans on the valid atoms, 0 on padding, in place, for x_a and (if not NULL) x_b with the same
 *     R and trans per set.  normals4 (n, 4): the standard normals the rotation quaternion is built from (:296-350);
 *     trans (n, 3) or NULL.
 *   kfb_sampler_prepare replaces _apply_forward_pinned_churn (ecsi.py:670-732) and the input preconditioning of
 *     inference_step (:624-633): x_hat = a x_t + b x_T + c noise (noise counted as zero on padding atoms; with noise = NULL
 *     the step does not churn and x_hat = x_t), r6 = [c_in x_hat | x_T * inv_sigma_T] (n, l, 6), the score network's input.
 *   kfb_sampler_update replaces the output preconditioning (:666-667), custom_rigid_align(..., rotation_only=True) (:59-103,
 *     :535), do_centering (:538) and _update_step (:734-807): x0 = c_skip x_noisy + c_out r_update, rotated onto x_noisy
 *     over the valid atoms, centred on them, zero on padding; x_next = ca x_noisy + cb x0 + cc x_T + cd noise (noise = NULL:
 *     the deterministic SI update).  x0_hat (n, l, 3) or NULL receives the aligned, centred estimate.
 *   kfb_rigid_align replaces custom_rigid_align with output_mask = mask (ecsi.py:59-103; the weighted Kabsch fit of
 *     src/kfold/utils/geometry/rigid_align.py:685-771, computed from the 3 x 3 covariance through the largest eigenvector
 *     of Horn's 4 x 4 matrix instead of an SVD: the same proper rotation).
 *   kfb_center_coords replaces do_centering (random_augment.py:90-130): subtract the mean of the valid atoms, zero padding.
 */
KFB_API int kfb_coords_augment(float* x_a, float* x_b, const float* normals4, const float* trans, const unsigned char* mask, int n,
                               int l, int mask_div, void* stream);
KFB_API int kfb_sampler_prepare(const float* x_t, const float* x_T, const float* noise, const unsigned char* mask, float a, float b,
                                float c, float c_in, float inv_sigma_T, float* x_hat, float* r6, int n, int l, int mask_div,
                                void* stream);
KFB_API int kfb_sampler_update(const float* x_noisy, const float* r_update, const float* x_T, const float* noise,
                               const unsigned char* mask, float c_skip, float c_out, float ca, float cb, float cc, float cd,
                               float* x_next, float* x0_hat, int n, int l, int mask_div, void* stream);
KFB_API int kfb_rigid_align(const float* coords, const float* target, const unsigned char* mask, int rotation_only, float* out, int n,
                            int l, int mask_div, void* stream);
KFB_API int kfb_center_coords(const float* coords, const unsigned char* mask, float* out, int n, int l, int mask_div, void* stream);

/*
 * Transition: out = Linear_out(silu(u_a) * u_b), [u_a, u_b] = Linear(LayerNorm(x))  (+ resid).
 * Replaces Transition.forward (src/kfold/model/layers/folding/transition.py:48-68) with SwiGLU.forward
 * (src/kfold/model/primitives/activation.py:27-29).
 *   x, out : (rows, c) of `dtype`;  w_swiglu_packed : bf16 [2*hidden, c], the silu half and the linear
 *   half interleaved in blocks of 128 rows, the silu half multiplied by 0.5 (exact in bf16: silu(a) = a' + a' tanh(a'),
 *   a' = a / 2; unscaled with KFB_FP32_PRECISE);  w_out : bf16 [c, hidden];  hidden a multiple of 128.
 */
KFB_API size_t kfb_transition_workspace_bytes(long long rows, int c, int hidden);
KFB_API size_t kfb_transition_workspace_bytes_precise(long long rows, int c, int hidden);
KFB_API int kfb_transition_fwd(const void* x, const float* ln_w, const float* ln_b, const void* w_swiglu_packed,
                               const void* w_out, void* out, const void* resid, void* workspace, size_t workspace_bytes,
                               long long rows, int c, int hidden, float eps, int dtype, void* stream);


/*
 * Transition for callers that cannot provide scratch memory (no counterpart in the reference).
 * Same arguments and result as kfb_transition_fwd minus the workspace: the two temporaries live in
 * a fixed 8 MiB device array inside the library (kfb_transition_static_max_bytes()), which every
 * GPU that loads the library holds until the process exits.  Meant for hosts where device
 * allocation is off-limits while they run -- a server whose memory pool was sized and frozen at
 * start-up, or a plugin callback that must not call cudaMalloc because it synchronises the device.
 * The function itself allocates nothing on the device or through any library.
 *   - Sizes whose temporaries exceed the array (rows * (c + hidden) * 2 bytes, each part rounded up
 *     to 256; six times that with dtype = KFB_FP32_PRECISE) are refused with KFB_ERR_UNSUPPORTED and
 *     a message naming the limit; e.g. c=384, hidden=1536 fits up to 2184 rows (364 in the
 *     fp32-accurate mode).
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call outside any stream capture.
 *   - All calls on a device share the one array: calls that may overlap on the GPU (different
 *     streams without ordering) race on it.  Nothing needs clearing between calls -- the
 *     temporaries are fully rewritten before use.
 */
KFB_API size_t kfb_transition_static_max_bytes(void);
KFB_API int kfb_transition_fwd_static(const void* x, const float* ln_w, const float* ln_b, const void* w_swiglu_packed,
                                      const void* w_out, void* out, const void* resid, long long rows, int c, int hidden,
                                      float eps, int dtype, void* stream);

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
