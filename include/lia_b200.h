/*
 * lia_b200.h -- C ABI of libliab200.so: the B200 (sm_100a) kernels behind LIA's OPT
 * decoder-layer hot path.
 *
 * Boundary rules:
 *   - plain pointers and sizes only; every device pointer is owned by the caller
 *     (PyTorch on the Python side) -- the library never allocates or frees device
 *     memory behind the caller's back;  the only allocations it owns are the ones made
 *     explicitly through the functions below: pinned host arenas, streamer handles and
 *     the peer-mappable device arenas of the tensor-parallel path (lia_p2p_*).
 *   - all work is enqueued on the stream that is passed in; no hidden
 *     synchronisation (contrast lia/modeling_opt.py:1339 torch.cuda.synchronize()).
 *   - no C++ exceptions cross the ABI.  Functions return 0 on success, a negative
 *     LIA_ERR_* code on failure; lia_last_error() returns the message of the last
 *     failure on the calling thread.  (The reference's only C ABI,
 *     lia/cxl/numa_alloc.c:29-33,47-55, signals failure with NULL + stderr; its Python
 *     side raises MemoryError, lia/modeling_opt.py:175.)
 *   - bf16 storage, fp32 accumulation everywhere; rounding points mirror the
 *     reference's eager op sequence.
 *
 * Each entry point names the reference interface it replaces (paths relative to the
 * reference root;  D = intel_extension_for_pytorch/transformers/models/reference/modules/decoder.py,
 * A = .../modules/attentions.py, M = lia/modeling_opt.py).
 */
#ifndef LIA_B200_H_
#define LIA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LIA_ABI_VERSION 9

typedef void* lia_stream_t; /* cudaStream_t */

enum {
  LIA_OK = 0,
  LIA_ERR_INVALID = -1, /* bad argument / unsupported shape */
  LIA_ERR_CUDA = -2,    /* a CUDA runtime/driver call failed */
  LIA_ERR_NOMEM = -3,   /* pinned host allocation failed */
  LIA_ERR_ARCH = -4     /* device is not sm_100 */
};

/* GEMM epilogues.  All start from r1 = bf16(acc_fp32), r2 = bf16(r1 + bias)  (two
 * roundings, as `torch.matmul(x, w.t()) + b` produces: A:393-394,418; D:62,81,88,94). */
enum {
  LIA_EPI_BIAS = 0,          /* out = r2                                   q/k/v style, D:81 */
  LIA_EPI_BIAS_RELU = 1,     /* out = relu(r2)                             fc1, D:92-105 */
  LIA_EPI_BIAS_RESIDUAL = 2, /* out = bf16(residual + r2)                  out_proj/fc2 + D:229,310 */
  LIA_EPI_QKV = 3            /* fused q|k|v projection, see LiaQkvArgs     A:376-418,456-491 */
};

/* Fused QKV projection epilogue.  W is [3*hq, K] = rows of Wq, then Wk, then Wv (hq = local
 * attention width, h or h/TP);  A is [B*S, K] with row m = b*S + s.
 *   columns [0,hq)    -> q_out[m, c]                = bf16(r2 * q_scale)        (A:418, A:456)
 *   columns [hq,2hq)  -> k_cache[pos0+s, b0+b, c]   = r2                        (A:393, A:457-491)
 *   columns [2hq,3hq) -> v_cache[pos0+s, b0+b, c]   = r2                        (A:394)
 * caches are time-major [Tmax, cache_batch, hq] (the reference's [(S+new),B,H,d], A:471-472). */
typedef struct LiaQkvArgs {
  void* q_out;
  void* k_cache;
  void* v_cache;
  int32_t hq;
  int32_t S;           /* tokens per sequence in this call (1 in decode) */
  int32_t pos0;        /* first cache row to write (= tokens already cached) */
  int32_t cache_batch; /* batch dimension of the cache tensors */
  int32_t b0;          /* batch offset of this minibatch inside the cache */
  float q_scale;       /* head_dim ** -0.5, M:413 */
} LiaQkvArgs;

int lia_abi_version(void);
const char* lia_last_error(void);
/* sm count / compute capability of the current device. */
int lia_device_info(int* sm_count, int* cc_major, int* cc_minor);

/* LayerNorm over the last dim: bf16 in, fp32 statistics, bf16 out.
 * Replaces gpu_ln_compute_self_attn / gpu_ln_compute_final (D:107-119) and the decoder's
 * final_layer_norm (M:1563-1564).  h % 8 == 0, h <= 16384. */
int lia_layernorm_bf16(const void* x, const void* w, const void* b, void* y, int rows, int h, float eps,
                       lia_stream_t stream);

/* out[M,N] = epilogue(A[M,K] . W[N,K]^T): tcgen05/TMEM GEMM fed by TMA.
 * Replaces gpu_linear_compute* / gpu_linear_relu_compute* (D:79-105) and the three
 * projections of A:376-418.  A, W, bias, residual, out are bf16 row-major and contiguous
 * (K % 8 == 0, N % 8 == 0, all base pointers 16-byte aligned).
 * `workspace` is used when the kernel splits K (small M): lia_gemm_workspace_bytes() bytes,
 * zero-initialised ONCE by the caller (the kernel leaves it zeroed again). */
size_t lia_gemm_workspace_bytes(int M, int N, int K);
int lia_gemm_bf16(const void* A, const void* W, const void* bias, const void* residual, void* out, int M, int N,
                  int K, int epilogue, const LiaQkvArgs* qkv, void* workspace, size_t workspace_bytes,
                  lia_stream_t stream);

/* Causal self-attention over a prompt (prefill), replaces A:444-449,493-536 for tgt_len > 1.
 * q [B,S,H,d] (already scaled), k/v caches [Tmax, cache_batch, H, d] holding rows [0,S) of
 * sequences b0..b0+B-1;  out [B,S,H*d].  Scores are rounded to bf16, softmax in fp32,
 * probabilities rounded to bf16 before P.V (A:499,512,529).  d in {64,128}. */
int lia_attn_prefill_bf16(const void* q, const void* k_cache, const void* v_cache, void* out, int B, int H, int S,
                          int d, int cache_batch, int b0, lia_stream_t stream);

/* Decode attention: one query token per sequence over T cached positions (the new token's
 * K/V row already written), NO mask (A:500).  Flash-decoding: `splits` > 1 partitions T over
 * CTAs and combines through `workspace` (lia_attn_decode_workspace_bytes()); splits == 0 lets
 * the library choose (aiming for 2 CTAs per SM), splits == -n lets it choose aiming for n CTAs
 * per SM (a tensor-parallel rank that keeps few heads).  q [B,H,d], out [B,H*d]. */
size_t lia_attn_decode_workspace_bytes(int B, int H, int d, int max_splits);
int lia_attn_decode_bf16(const void* q, const void* k_cache, const void* v_cache, void* out, int B, int H, int T,
                         int d, int cache_batch, int b0, int splits, void* workspace, size_t workspace_bytes,
                         lia_stream_t stream);

/* Stand-alone Q scaling + KV-cache append for callers that hold separate q/k/v [B,S,hq] (the
 * IndirectAccessKVCache operator face, llm/modules/mha_fusion.py:503-560); the model path fuses this
 * into the QKV GEMM epilogue.  q_out = bf16(q*q_scale); caches as in LiaQkvArgs (A:456-491). */
int lia_kv_append_bf16(const void* q, const void* k, const void* v, void* q_out, void* k_cache, void* v_cache, int B,
                       int S, int hq, int pos0, int cache_batch, int b0, float q_scale, lia_stream_t stream);

/* hidden[b,s,:] = embed_tokens[ids[b,s]] + embed_positions[past_len + s + 2]  (M:1107-1142 with
 * an all-ones attention mask, M:368-378).  ids int64 [B,S].  Either table (not both) may be NULL: its rows
 * then contribute nothing and the other table's rows are copied through -- opt-350m's project_in path looks
 * token rows [word_embed_proj_dim] and position rows [hidden] up separately (M:1139-1142). */
int lia_embed_bf16(const int64_t* ids, const void* embed_tokens, const void* embed_positions, void* out, int B,
                   int S, int h, int past_len, int vocab, int max_pos_rows, lia_stream_t stream);

/* The same with the positions OPTLearnedPositionalEmbedding.forward derives from an attention mask
 * (M:368-378): p = cumsum(mask[b,:])[past_len+s] * mask[b,past_len+s] - 1, row = p + 2.  attention_mask
 * is int64 [B, mask_ld] with mask_ld >= past_len + S (HF's mask covers past and current tokens,
 * M:1127-1131); NULL means all ones.  Padded prompts change ONLY the positions on the reference's GPU
 * branch: its attention rebuilds a pure causal mask in prefill and applies none in decode (A:446-449, A:500). */
int lia_embed_masked_bf16(const int64_t* ids, const int64_t* attention_mask, int mask_ld, const void* embed_tokens,
                          const void* embed_positions, void* out, int B, int S, int h, int past_len, int vocab,
                          int max_pos_rows, lia_stream_t stream);

/* next[b] = argmax_v logits[b, v] with logits[b, suppress_id] treated as -inf when
 * suppress_id >= 0 (min_new_tokens processor, lia/generation_utils.py:872-880; argmax at
 * intel_extension_for_pytorch/transformers/generation/greedy_search.py:395).  Lowest index
 * wins ties (torch.argmax on CPU).  logits bf16 [B,V], next int64 [B]. */
int lia_argmax_bf16(const void* logits, int64_t* next, int B, int V, int suppress_id, lia_stream_t stream);

/* out = bf16(residual + x): the residual add that follows the all-reduce of a row-parallel
 * projection under tensor parallelism (D:247, D:317; the reduce itself replaces D:60-68).
 * n = number of elements, n % 8 == 0. */
int lia_residual_add_bf16(const void* x, const void* residual, void* out, size_t n, lia_stream_t stream);

/* ---- tensor parallelism: row-parallel projection FUSED with its all-reduce and residual add.
 *
 * Replaces, for world > 1, the reference's  GPU GEMM -> .to('cpu') -> deepspeed_comm.all_reduce
 * (oneCCL) -> .to('cuda') -> residual add  chain (gpu_linear_allreduce_compute D:60-77, then
 * D:247 / D:317) with ONE kernel that exchanges partial tiles over NVLink peer memory while the
 * remaining tiles are still being computed:
 *     out = bf16( residual + bf16( sum_r  bf16( bf16(acc_r) + bias_r ) ) )
 * (bias_r is this rank's share of the bias, i.e. bias / world, tensor_parallel.py:134; the sum over
 * ranks is taken in fp32 in rank order, so every rank produces bit-identical results).
 *   M <= 128 (decode), world < 4: one-shot -- the CTA that finishes an output tile pushes it into
 *     every peer's receive area as {4 data bytes, epoch} words (data and validity arrive together:
 *     one one-way NVLink latency, no fence, no flag), then reduces the `world` partials in its own.
 *   M <= 128 (decode), world >= 4: two-shot with per-row ownership -- row group `it` of tile `ta` is
 *     reduced by rank (it + ta) % world, so every thread on every rank reduces 1/world of its own
 *     values and receives the rest as finals in the same {data, epoch} framing: two one-way
 *     latencies, 2(world-1)/world x the data per rank instead of (world-1) x.
 *   M >  128 (prefill): two-shot -- tile u is owned by rank u % world; the other ranks push their
 *     partial to the owner, which reduces, adds the residual and writes the final tile into every
 *     rank's `out` (which therefore must live inside the arena, at the same offset on every rank);
 *     flags trail their data by one tile so no warp ever waits out an NVLink round trip.  With a multicast
 *     mapping of the arena (LiaTpArgs.mc_arena) the reduction happens inside the NVLink switch instead.
 * All cross-GPU traffic goes through one symmetric "arena" per rank (lia_p2p_alloc), mapped into
 * every peer with CUDA IPC.  Every rank must issue the same sequence of calls with the same shapes.
 * Launches are safe under CUDA-graph replay (epochs live in device memory).  A peer that does
 * not show up within LIA_TP_TIMEOUT_NS makes the kernel give up and set the arena's error word
 * (lia_tp_error) instead of hanging the GPU. */
#define LIA_TP_MAX_WORLD 8
#define LIA_TP_MAX_UNITS 16384   /* output tiles per call */
typedef struct LiaTpArgs {
  int32_t rank, world;
  void* arena[LIA_TP_MAX_WORLD]; /* arena[r] = rank r's arena mapped in this process; arena[rank] is local */
  uint64_t ctl_off;              /* lia_tp_ctl_bytes() bytes, zero-initialised once (epoch, flags)      */
  uint64_t recv_off;             /* receive area: 2 * recv_bytes (two parities)                          */
  uint64_t recv_bytes;           /* >= lia_tp_recv_bytes(M, N, K, world)                                 */
  uint64_t out_off;              /* M > 128 only: offset of `out` inside the arena                       */
  void* mc_arena;                /* NVLink-switch MULTICAST address of the same arena (every rank's copy behind one
                                  * address), or NULL.  When set, the prefill exchange (M > 128) reduces INSIDE the switch:
                                  * ranks keep their partial tiles in their own arena, the owner of a tile reads the sum of
                                  * all copies with multimem.ld_reduce and writes the final tile to every rank with one
                                  * multimem.st -- ~1.1 S instead of 1.75 S bytes per rank and 7x fewer SM-issued remote
                                  * accesses.  The arena must then be symmetric memory bound to a multicast object
                                  * (torch.distributed._symmetric_memory; tp.SymmArena). */
} LiaTpArgs;
size_t lia_tp_ctl_bytes(void);
size_t lia_tp_recv_bytes(int M, int N, int K, int world);
int lia_gemm_allreduce_bf16(const void* A, const void* W, const void* bias, const void* residual, void* out, int M,
                            int N, int K, const LiaTpArgs* tp, void* workspace, size_t workspace_bytes,
                            lia_stream_t stream);
/* reads (and clears) the arena's error word: 0 = ok, 1 = a peer timed out.  Synchronises the device. */
int lia_tp_error(const LiaTpArgs* tp);

/* peer-mappable device memory (cudaMalloc + CUDA IPC).  lia_p2p_alloc zero-fills the buffer and
 * writes a 64-byte handle that another PROCESS passes to lia_p2p_open to map it. */
#define LIA_P2P_HANDLE_BYTES 64
int lia_p2p_alloc(size_t bytes, void** dev_ptr, void* handle_out);
int lia_p2p_open(const void* handle, void** peer_ptr);
int lia_p2p_close(void* peer_ptr);
int lia_p2p_free(void* dev_ptr);

/* ---- pinned host arena: replaces lia/cxl/numa_alloc.c (numa_alloc_node / numa_free_node) and
 * pin_memory (M:167-227).  Returns NULL on failure (message in lia_last_error()). */
void* lia_host_arena_alloc(size_t bytes);
int lia_host_arena_free(void* ptr, size_t bytes);

/* ---- layer streamer: double-buffered H2D of non-resident layers on a private copy stream.
 * Replaces load_layer / layer_copy (M:270-318) and the stream/event choreography of
 * M:1208-1212,1288-1316.  The caller owns the device slabs (n_slots buffers of slab_bytes). */
typedef struct LiaStreamer LiaStreamer;
LiaStreamer* lia_streamer_create(void* const* device_slabs, int n_slots, size_t slab_bytes);
/* enqueue host_src[0:bytes] -> slot on the copy stream, after all compute previously recorded
 * as using that slot (lia_streamer_release) has finished. */
int lia_streamer_prefetch(LiaStreamer* s, int slot, const void* host_src, size_t bytes);
/* make `compute_stream` wait until the last prefetch into `slot` has landed. */
int lia_streamer_wait(LiaStreamer* s, int slot, lia_stream_t compute_stream);
/* record on `compute_stream` that the slot's contents are no longer needed after this point. */
int lia_streamer_release(LiaStreamer* s, int slot, lia_stream_t compute_stream);
/* total bytes copied and device-measured copy milliseconds since creation (blocks on the copy stream). */
int lia_streamer_stats(LiaStreamer* s, double* bytes, double* copy_ms);
int lia_streamer_destroy(LiaStreamer* s);

/* ---- decode programs: a chain of decode-shaped operations (at most 128 token rows each) executed as ONE persistent
 * kernel -- what a decode step of the reference spends ~30 library launches per layer on (lia/modeling_opt.py:1379-1491
 * driving decoder.py:172-335 and attentions.py:312-557; models.py:423-431 and greedy_search.py:367-395 for the head).
 * Operations run in the order they were added; each starts when all earlier ones are complete on every SM, while the
 * weight tiles of later GEMMs and the cached K/V rows of later attention operations already stream into shared memory.
 * Every operation computes exactly what its stand-alone entry point computes (same kernels' code, same summation order):
 * results are bit-identical to calling lia_layernorm_bf16 / lia_gemm_bf16 / lia_gemm_allreduce_bf16 /
 * lia_attn_decode_bf16 (splits == 1) / lia_embed_masked_bf16 / lia_argmax_bf16 one after the other.
 * All pointers are device pointers owned by the caller and must stay valid until lia_program_destroy. */
typedef struct LiaProgram LiaProgram;
LiaProgram* lia_program_create(int rows);                       /* rows = token rows (1..128) of every operation */
int lia_program_add_layernorm(LiaProgram* p, const void* x, const void* w, const void* b, void* y, int rows, int h, float eps);
/* as lia_gemm_bf16 (tp == NULL) or lia_gemm_allreduce_bf16 (tp != NULL; `epilogue` ignored).  A LIA_EPI_QKV
 * epilogue appends at the position given to lia_program_run (qkv->pos0 is ignored). */
int lia_program_add_gemm(LiaProgram* p, const void* A, const void* W, const void* bias, const void* residual, void* out, int M,
                         int N, int K, int epilogue, const LiaQkvArgs* qkv, const LiaTpArgs* tp);
/* as lia_attn_decode_bf16 with T = pos0 + 1 of the run; cache_rows = rows the cache tensors have */
int lia_program_add_attn_decode(LiaProgram* p, const void* q, const void* k_cache, const void* v_cache, void* out, int B, int H,
                                int d, int cache_batch, int b0, int cache_rows);
/* as lia_embed_masked_bf16 with S = 1, past_len = pos0 and ids = the run's ids_in */
int lia_program_add_embed(LiaProgram* p, const int64_t* attention_mask, int mask_ld, const void* embed_tokens,
                          const void* embed_positions, void* out, int B, int h, int vocab, int max_pos_rows);
/* as lia_argmax_bf16 into the run's ids_out, with the run's suppress_id */
int lia_program_add_argmax(LiaProgram* p, const void* logits, int B, int V);
int lia_program_finalize(LiaProgram* p);                        /* uploads the program; no more operations after it */
/* one launch: pos0 = positions already cached (the new token is appended at pos0 and attends to pos0 + 1 keys) */
int lia_program_run(LiaProgram* p, int pos0, const int64_t* ids_in, int64_t* ids_out, int suppress_id, lia_stream_t stream);
int lia_program_error(LiaProgram* p);                           /* 0 = ok, 1 = a CTA timed out; synchronises the device */
int lia_program_num_ops(LiaProgram* p);
int lia_program_destroy(LiaProgram* p);

/* ------------------------------------------------------------------------------------------------------------------
 * Models with a 32-bit residual stream, recurrent (matrix-memory) mixers and latent-cache attention.
 * Flags `*_f32` say whether a buffer holds fp32 (1) or bf16 (0); norm weights, biases, gates, state and the residual
 * stream are always fp32.  `segs[s] = {slot, first position, first row, rows}` describes the portion of sequence `slot`
 * that occupies rows [first row, first row + rows) of the step; `meta[row] = {slot, position}` says the same per row.
 * The reference has none of these (its only model family is OPT). */

/* x[row] = w * e / sqrt(mean(e^2) + eps), e = table[ids[row]];  w_n = 1 (one number for all channels) or W */
int lia_embed_rmsnorm(const int64_t* ids, const void* table, int table_f32, const float* w, int w_n, float* x, int rows, int W,
                      int vocab, float eps, lia_stream_t stream);
/* y != NULL: x += w_post * y / rms(y) (norm after a sublayer + residual sum);  h != NULL: h = w_pre * x / rms(x) */
int lia_rms_add_norm(float* x, const void* y, int y_f32, const float* w_post, int w_post_n, const float* w_pre, int w_pre_n,
                     void* h, int h_f32, int rows, int W, float eps, lia_stream_t stream);
/* h[r] = w * x[rows[r]] / rms(x[rows[r]]) for n selected rows */
int lia_rms_gather(const float* x, const int* rows, const float* w, int w_n, void* h, int h_f32, int n, int W, float eps,
                   lia_stream_t stream);
/* out = g * sigmoid(alpha g) * (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit); gate_up rows hold gate at column 0 and up at column up_off */
int lia_clamped_glu(const void* gate_up, int ld, int up_off, void* out, int act_f32, int M, int F, float limit, float alpha, lia_stream_t stream);
/* out[m][n] = act(a[m] . w[n] + bias[n]), N small (per-head gates), fp32 out.  mode 0: identity; 1: first N/2 outputs
 * cap*tanh(z/cap), last N/2 logsigmoid(cap*tanh(z/cap)) (log input / log forget gates); 2: sigmoid */
int lia_linear_small(const void* a, int a_f32, int lda, const void* w, int w_f32, const float* bias, float* out, int M, int N, int K,
                     int mode, float cap, lia_stream_t stream);
/* C[b][m][n] = scale * sum_k A[b][m][k] W[b][n][k] on the CUDA cores, fp32 products and sums; element strides */
int lia_linear_plain(const void* A, int a_f32, long long lda, long long sA, const void* W, int w_f32, long long ldw, long long sW,
                     void* C, int c_f32, long long ldc, long long sC, int M, int N, int K, int batch, float scale, lia_stream_t stream);
int lia_argmax_f32(const float* logits, int64_t* next, int B, int V, int suppress_id, lia_stream_t stream);
/* matrix-memory recurrence over every portion of the step; q/k [rows][H*dim], v [rows][H*vdim] with row stride ld;
 * gates [rows][2H] = log input gates then log forget gates; state_S [slots][H][vdim][dim], state_n [slots][H][dim],
 * state_m [slots][H]; o [rows][H*vdim] = S^T q / (max(|n.q|, exp(-m)) + den_eps) */
int lia_mlstm_scan(const void* q, const void* k, const void* v, int act_f32, int ld, const float* gates, float* state_S, float* state_n,
                   float* state_m, const int* segs, int nseg, int H, int dim, int vdim, float q_scale, float den_eps, float* o,
                   lia_stream_t stream);
/* out[row][h] = o[row][h] / rms_over_vdim * w[h] * act(gate[row][h]), act = sigmoid (gate_silu == 0) or SiLU */
int lia_headnorm_gate(const float* o, const float* w, const void* gate, int ldg, void* out, int act_f32, int M, int H, int vdim, float eps,
                      int gate_silu, lia_stream_t stream);
/* cache[slot][pos] = [rmsnorm(dkv[:kv_rank]) * c_norm_w | rotate(dkv[kv_rank:], pos)];  qa[row][h][kv_rank:] =
 * rotate(q[row][h][dim:], pos)  (qa rows are [H][kv_rank + rot] fp32; the caller fills qa[..][:kv_rank]) */
int lia_latent_prep(const void* q, int ldq, const void* dkv, int ldd, int act_f32, const float* c_norm_w, const float* inv_freq,
                    const int* meta, void* cache, long long slot_stride, float* qa, int M, int H, int dim, int rot, int rot_dims,
                    int kv_rank, float eps, lia_stream_t stream);
/* out[row][h] = gate[row][h] * sum_{s <= pos(row)} softmax_s((qa[row][h] . cache[slot][s]) * scale) cache[slot][s][:kv_rank]
 * (gate may be NULL: no output gate).  nsplit > 1 splits every row's keys over nsplit blocks (decoding over a long history);
 * it needs a workspace of lia_latent_attn_workspace_floats(...) floats and runs a second, combining kernel. */
size_t lia_latent_attn_workspace_floats(int M, int H, int kv_rank, int nsplit);
int lia_latent_attn(const float* qa, const void* cache, int cache_f32, long long slot_stride, const int* meta, const float* gate,
                    float* out, float* workspace, int nsplit, int M, int H, int kv_rank, int rot, float scale, lia_stream_t stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Models whose sublayers sit between layer norms (weight and bias) on a 32-bit residual stream, with linear-attention
 * recurrences (a fixed decay per head, or the gated delta rule behind a short convolution), sliding-window attention
 * with grouped key/value heads, and dense or mixture-of-experts feed-forwards.  Same conventions as the section above.
 * The reference has none of these. */
enum { LIA_ACT_NONE = 0, LIA_ACT_RELU = 1, LIA_ACT_SILU = 2, LIA_ACT_GELU_ERF = 3, LIA_ACT_GELU_TANH = 4,
       LIA_ACT_CLAMPED_SWISH = 5 /* gated form only: see lia_moe_gemm_act */ };

/* x[r] = table[ids[r]] as fp32; x_copy (may be NULL) receives the same rows */
int lia_embed_rows(const int64_t* ids, const void* table, int table_f32, float* x, float* x_copy, int rows, int W, int vocab,
                   lia_stream_t stream);
/* if y: x += mult * (LN(y) * w_post + b_post);  if extra: x += extra;  if h: h = LN(x) * w_pre + b_pre.
 * LN(z) = (z - mean) / sqrt(mean((z - mean)^2) + eps), fp32. */
int lia_ln_add_norm(float* x, const void* y, int y_f32, const float* w_post, const float* b_post, float mult, const float* extra,
                    const float* w_pre, const float* b_pre, void* h, int h_f32, int rows, int W, float eps, lia_stream_t stream);
int lia_ln_gather(const float* x, const int* rows, const float* w, const float* b, void* h, int h_f32, int n, int W, float eps,
                  lia_stream_t stream);
/* out[m][f] = act(in[m][f]) * in[m][up_off + f]; up_off < 0: out = act(in).  `in` has row stride ld. */
int lia_gated_act(const void* in, int ld, int up_off, void* out, int act_f32, int M, int F, int act, lia_stream_t stream);

/* softmax over E fp32 logits per row, the `top` largest (lowest index first on ties), divided by their sum + 1e-20 */
int lia_router_topk(const float* logits, int* idx, float* wt, int M, int E, int top, lia_stream_t stream);
/* the same with a per-expert correction (may be NULL) added to the scores for the CHOICE only, and the weights = the chosen
 * experts' plain scores, divided by their sum + 1e-20 only if renorm != 0 */
int lia_router_topk_ext(const float* logits, const float* correction, int renorm, int* idx, float* wt, int M, int E, int top,
                        lia_stream_t stream);
/* (token, choice) pairs grouped by expert into tiles of lia_moe_tile_rows() rows: perm[n_tiles * rows] (pair or -1),
 * tile_expert[n_tiles] (expert or -1), pos_of[pairs] (place of a pair in perm).
 * n_tiles >= (pairs + min(E, pairs) * (rows - 1)) / rows. */
int lia_moe_tile_rows(void);
int lia_moe_plan(const int* idx, int pairs, int E, int n_tiles, int* perm, int* tile_expert, int* pos_of, lia_stream_t stream);
/* One projection of every expert (weights [E][N][K], expert stride given) over its own rows.
 * up != 0: C[place of pair] = act(A[pair / top] @ W[e].T), C of the activations' type;
 * up == 0: C[pair] = wt[pair] * (A[place of pair] @ W[e].T), C fp32.
 * perm == NULL: the few-rows form; a pair's place is the pair itself and idx[pair] names its expert. */
int lia_moe_gemm(const void* A, int a_f32, int lda, const void* W, int w_f32, long long w_expert_stride, void* C, int c_f32, int ldc,
                 const int* perm, const int* tile_expert, int n_tiles, const int* idx, const float* wt, int pairs, int top, int N, int K,
                 int up, int act, lia_stream_t stream);
/* the same; gated != 0 (up only): W is [E][2N][K], N gate rows then N up rows, and C = act(gate sum) * (up sum); pairs and
 * tiles of experts >= n_real (experts without weights: lia_moe_combine_ext serves them) are skipped */
int lia_moe_gemm_ext(const void* A, int a_f32, int lda, const void* W, int w_f32, long long w_expert_stride, void* C, int c_f32, int ldc,
                     const int* perm, const int* tile_expert, int n_tiles, const int* idx, const float* wt, int pairs, int top, int N, int K,
                     int up, int act, int gated, int n_real, lia_stream_t stream);
/* dst[place] = src[perm[place] / top] (zeros where perm is -1): the experts' inputs in the plan's order */
int lia_moe_gather(const void* src, int act_f32, const int* perm, void* dst, int places, int W, int top, lia_stream_t stream);
/* C[rows of expert e] = A[rows of expert e] @ W[e].T (bf16, lia_gemm_bf16 per expert): expert e owns the next
 * tiles_per_expert[e] * tile_rows rows (tiles_per_expert is a HOST array); workspace as for lia_gemm_bf16 at the largest M. */
int lia_moe_expert_gemms(const void* A, const void* W, long long w_expert_stride, void* C, const int* tiles_per_expert, int E, int tile_rows,
                         int N, int K, void* workspace, size_t workspace_bytes, lia_stream_t stream);
/* y[m] = sum_t f(m * top + t) (+ shared[m], may be NULL), fp32; f(pair) = ypair[pair], or, when pos_of is given,
 * wt[pair] * ypair[pos_of[pair]] */
int lia_moe_combine(const void* ypair, int ypair_f32, const int* pos_of, const float* wt, const void* shared, int shared_f32, float* y, int M,
                    int W, int top, lia_stream_t stream);
/* the same with identity experts: a pair whose idx[pair] >= n_real contributes wt[pair] * h[m] (h: the experts' input, of the
 * activations' type like `shared`), and ypair is not read for it */
int lia_moe_combine_ext(const void* ypair, int ypair_f32, const int* pos_of, const float* wt, const void* shared, int act_f32, const int* idx,
                        int n_real, const void* h, float* y, int M, int W, int top, lia_stream_t stream);

/* Short causal convolution (taps <= 16, weights [channels][taps], last column = current token) + SiLU over the q | k | v
 * channels of a projection's output y (row stride ld, column offsets given; q and k have G heads of dim, v has H of vdim);
 * q and k divided by sqrt(sum of squares + unit_eps) per head, q times q_scale; gates [M][2H] hold W_b h | W_a h on entry and
 * beta = sigmoid(.) | g = exp(-exp(a_log) * softplus(. + dt_bias)) on return.  conv_state [slot][taps-1][channels] fp32 holds
 * the inputs before each portion; lia_conv_state_update (after lia_conv_prep or lia_qkv_prep) moves it past the step's portions
 * (nq, nk, nv channels of q, k, v at the given column offsets). */
int lia_conv_prep(const void* y, int y_f32, int ld, int q_off, int k_off, int v_off, const float* wconv, const float* conv_state,
                  const int* meta, float* gates, const float* a_log, const float* dt_bias, float* qk, float* v, int M, int G, int H,
                  int dim, int vdim, int taps, float q_scale, float unit_eps, lia_stream_t stream);
int lia_conv_state_update(const void* y, int y_f32, int ld, int q_off, int k_off, int v_off, int nq, int nk, int nv, float* conv_state,
                          const int* segs, int nseg, int taps, lia_stream_t stream);
/* Matrix-state recurrence over every portion; state_S [slot][H][vdim][dim] fp32, o [rows][H * vdim] fp32.
 * gates == NULL:  S = decay[h] S + k v^T, o = S^T q.   gates [rows][2H] = beta | g:  the gated delta rule
 * S = g S; u = beta (v - S^T k); S += k u^T; o = S^T q.   q, k: G heads (head h reads h / (H / G)), row stride ldqk;
 * in_silu != 0 applies SiLU to q, k, v as they are read. */
int lia_linear_scan(const void* q, const void* k, int ldqk, const void* v, int ldv, int act_f32, int in_silu, const float* decay,
                    const float* gates, float* state_S, const int* segs, int nseg, int H, int G, int dim, int vdim, float* o,
                    lia_stream_t stream);

/* keys as they are and values divided by their per-head root mean square (norm_values != 0) into the caches
 * [slot][capacity][G * dim] and [slot][capacity][G * vdim] at meta[row] = {slot, position} */
int lia_kv_store(const void* k, int ldk, const void* v, int ldv, int act_f32, const int* meta, void* kcache, long long k_slot_stride,
                 void* vcache, long long v_slot_stride, int M, int G, int dim, int vdim, float eps, int norm_values, lia_stream_t stream);
/* out[row][h] = sum_j softmax_j(cap(q[row][h] . k[j][h / (H/G)] * scale * temp[h])) v[j][h / (H/G)] over 0 <= pos - j < window,
 * cap(s) = softcap * tanh(s / softcap) (softcap <= 0: none).  A block takes rows_per_block consecutive rows and
 * heads_per_block query heads (<= 8; whole groups of H/G heads, or a divisor of one group), with
 * rows_per_block * heads_per_block <= 8 * lia_window_attn_pairs_per_warp(vdim) and lia_window_attn_smem_bytes(...) of shared
 * memory (<= 200 KB).  nsplit > 1 splits every row's keys over nsplit blocks; it needs a workspace of
 * lia_window_attn_workspace_floats(...) floats and runs a second, combining kernel. */
int lia_window_attn_pairs_per_warp(int vdim);
size_t lia_window_attn_smem_bytes(int heads_per_block, int kv_heads_per_block, int rows_per_block, int dim, int vdim);
size_t lia_window_attn_workspace_floats(int M, int H, int vdim, int nsplit);
int lia_window_attn(const void* q, int ldq, int act_f32, const void* kcache, long long k_slot_stride, const void* vcache,
                    long long v_slot_stride, const int* meta, const float* temp, void* out, float* workspace, int M, int H, int G, int dim,
                    int vdim, int window, float scale, float softcap, int heads_per_block, int rows_per_block, int nsplit,
                    lia_stream_t stream);
/* lia_window_attn with more in the score and on the way out (each pointer may be NULL): slopes[h] * (pos - j) is taken off the
 * (capped) score; exp(sink[h]) joins the softmax's denominator as a term without key or value; the output is multiplied by a
 * gate -- gate_mode 1: fp32 gate[row][h]; 2: sigmoid(gate[row][h * vdim + c]) of the activations' type with row stride ldg.
 * window <= 0: every row sees its whole history.  q_f32 != 0: the queries are fp32 whatever the caches' type. */
int lia_window_attn_ext(const void* q, int ldq, int q_f32, int act_f32, const void* kcache, long long k_slot_stride, const void* vcache,
                        long long v_slot_stride, const int* meta, const float* temp, const float* slopes, const float* sink, const void* gate,
                        int gate_mode, int ldg, void* out, float* workspace, int M, int H, int G, int dim, int vdim, int window, float scale,
                        float softcap, int heads_per_block, int rows_per_block, int nsplit, lia_stream_t stream);
/* What turns the q | k | v columns of a projection's output y (row stride ld) into attention inputs, per token row with
 * meta[row] = {slot, position}; each step is optional and they come in this order:
 *   bias [H*dim + G*dim + G*vdim] added;
 *   a short causal convolution along the sequence, channel by channel (taps <= 16, wconv [channels][taps], last column = current token; the
 *   taps - 1 outputs of the projection before a portion come from conv_state [slot][taps-1][channels] fp32, kept current by
 *   lia_conv_state_update; what lies before the sequence's start is zero);
 *   RMS norm of q and of k -- norm_mode 1: over the whole projection, weights [H*dim] and [G*dim]; 2: per head, weights [dim];
 *   q times 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1) (temp_every > 0);
 *   rotation of the first rot_dims channels of every q and k head by pos * freq[i] (freq: rot_dims/2 doubles), pairs
 *   (2i, 2i+1), or (i, i + rot_dims/2) if rot_halves != 0; cos and sin times rot_mag;
 *   values -- vmix_mode 1: copied to v_first [M][G*vdim] fp32; 2: v moves towards v_first by the fraction lambda, v += lambda (v_first - v).
 * q goes to q_out [M][H*dim] fp32, k and v to the caches [slot][capacity][G*dim | G*vdim] of the activations' type. */
int lia_qkv_prep(const void* y, int act_f32, int ld, int q_off, int k_off, int v_off, const float* bias, const float* wconv,
                 const float* conv_state, int taps, int norm_mode, const float* qnorm_w, const float* knorm_w, float eps, float temp_coef,
                 int temp_every, const double* freq, int rot_dims, int rot_halves, float rot_mag, int vmix_mode, float lambda, float* v_first,
                 const int* meta, float* q_out, void* kcache, long long k_slot_stride, void* vcache, long long v_slot_stride, int M, int H,
                 int G, int dim, int vdim, lia_stream_t stream);

/* x_new = x + w * g / sqrt(mean(g^2) + eps) with g = y * sigmoid(r + rb) (r, rb may be NULL: no gate; y NULL: nothing added;
 * r has row stride ldr and the activations' type).  stack == NULL: x = x_new.  Else stack[n_mix - 1] = x_new and
 * x = sum_{j < n_mix} mix[j] * stack[j] (stack: [n][rows][W] fp32 with the given stride between entries).  h (may be NULL)
 * receives x in the activations' type. */
int lia_gated_rms_add(float* x, const void* y, int y_f32, const void* r, int ldr, const float* rb, const float* w, float* stack,
                      long long stack_stride, int n_mix, const float* mix, void* h, int act_f32, int rows, int W, float eps,
                      lia_stream_t stream);
/* out[m] = k1 R(z) + k2 R(z*z) + k3 R(z*z*z) + k0 over z = in[m][:F] (row stride ld), products element by element,
 * R(u) = u / sqrt(mean(u^2) + eps); coef = {k1, k2, k3, k0} fp32 on the device */
int lia_poly_norm(const void* in, int ld, const float* coef, void* out, int act_f32, int M, int F, float eps, lia_stream_t stream);

/* ---- Pre-norm designs with learned positions: latent attention with latent queries and a pairwise rotation, several attention
 * maps over shared values under a chunked mask, a forget-gate recurrence, experts with a clamped gated activation.  (ABI 9) ---- */

/* x[row] = table[ids[row]] * scale + pos_table[meta[row].position] in fp32 (pos_table may be NULL; the tables share a type).
 * cat (may be NULL): [rows][2 W] of the given type receives the row twice, side by side. */
int lia_embed_scale_pos(const int64_t* ids, const void* table, const void* pos_table, int table_f32, float scale, const int* meta, float* x,
                        void* cat, int cat_f32, int rows, int W, int vocab, int max_pos, lia_stream_t stream);
/* x = (replace ? 0 : x) + y + bias (y [rows][W], bias [W] fp32; each may be NULL), then h = w * x / sqrt(mean(x^2) + eps) in the
 * activations' type with row stride ldh (w NULL: h = x; h NULL: no output).  x is the fp32 residual stream. */
int lia_residual_norm(float* x, const void* y, int y_f32, int replace, const float* bias, const float* w, void* h, int h_f32, long long ldh,
                      int rows, int W, float eps, lia_stream_t stream);
/* out[m] = w * z / sqrt(mean(z^2) + eps), z = in[m][0..N) with row stride ld; out contiguous [M][N] */
int lia_rms_norm_rows(const void* in, int in_f32, long long ld, const float* w, void* out, int out_f32, int M, int N, float eps,
                      lia_stream_t stream);
/* out = a * sigmoid(gate) over [M][F]; a and gate are row-major views; out contiguous, of the gate's type */
int lia_sigmoid_mul(const void* a, int a_f32, long long lda, const void* gate, int gate_f32, long long ldg, void* out, int out_f32, int M, int F,
                    lia_stream_t stream);
/* x = cap * tanh(x / cap) in place over n numbers */
int lia_softcap_f32(float* x, long long n, float cap, lia_stream_t stream);
/* lia_moe_gemm_ext with the activation's parameters: LIA_ACT_CLAMPED_SWISH (gated up projection only) computes
 * g' * sigmoid(p1 * g') * (u' + 1) with g' = min(g, p0), u' = clamp(u, -p0, p0) */
int lia_moe_gemm_act(const void* A, int a_f32, int lda, const void* W, int w_f32, long long w_expert_stride, void* C, int c_f32, int ldc,
                     const int* perm, const int* tile_expert, int n_tiles, const int* idx, const float* wt, int pairs, int top, int N, int K,
                     int up, int act, int gated, int n_real, float act_p0, float act_p1, lia_stream_t stream);
/* The q | f | v columns of a projection's output -> fp32 inputs of the forget-gate recurrence: out[row] = silu(q) | low + (1 - low) *
 * sigmoid(f + f_bias) | v  (nq channels of q and of f, nv of v; f_bias may be NULL). */
int lia_forget_gate_prep(const void* y, int y_f32, int ld, int q_off, int f_off, int v_off, const float* f_bias, const float* low, float* out,
                         int M, int nq, int nv, lia_stream_t stream);
/* per head and channel d: S[d][:] <- f[d] S[d][:] + (1 - f[d]) v, then o = sum_d q[d] S[d][:], over every portion; state_S [slot][H][vdim][dim] fp32 (lia_linear_scan's layout) */
int lia_forget_scan(const float* q, const float* f, int ldqf, const float* v, int ldv, float* state_S, const int* segs, int nseg, int H, int dim,
                    int vdim, float* o, lia_stream_t stream);
/* lia_window_attn_ext with: chunk > 0 -- a query at position p attends to keys [p - p % chunk, p] only; v_div -- key head g
 * reads value head g / v_div (the value cache holds G / v_div heads); out_f32 -- fp32 output on caches of any type */
int lia_window_attn_masked(const void* q, int ldq, int q_f32, int act_f32, const void* kcache, long long k_slot_stride, const void* vcache,
                           long long v_slot_stride, const int* meta, const float* temp, const float* slopes, const float* sink, const void* gate,
                           int gate_mode, int ldg, void* out, int out_f32, float* workspace, int M, int H, int G, int v_div, int dim, int vdim,
                           int window, int chunk, float scale, float softcap, int heads_per_block, int rows_per_block, int nsplit,
                           lia_stream_t stream);
/* lia_qkv_prep with Gv value heads beside G key heads */
int lia_qkv_prep_heads(const void* y, int act_f32, int ld, int q_off, int k_off, int v_off, const float* bias, const float* wconv,
                       const float* conv_state, int taps, int norm_mode, const float* qnorm_w, const float* knorm_w, float eps, float temp_coef,
                       int temp_every, const double* freq, int rot_dims, int rot_halves, float rot_mag, int vmix_mode, float lambda, float* v_first,
                       const int* meta, float* q_out, void* kcache, long long k_slot_stride, void* vcache, long long v_slot_stride, int M, int H,
                       int G, int Gv, int dim, int vdim, lia_stream_t stream);
/* a [M][G][2][H/G][vdim] fp32 (two attention maps per head) -> out [M][H][vdim]: o = a1 - lambda a2, out = mult * o / sqrt(mean(o^2) + eps) */
int lia_diff_combine(const float* a, void* out, int act_f32, int M, int H, int G, int vdim, float lambda, float mult, float eps,
                     lia_stream_t stream);
/* lia_latent_prep with the rotation of channel pairs (2i, 2i+1) by pos * freq[i] (rot_dims/2 doubles) and the amplitude mag */
int lia_latent_prep_pairs(const void* q, int ldq, const void* dkv, int ldd, int act_f32, const float* c_norm_w, const double* freq, float mag,
                          const int* meta, void* cache, long long slot_stride, float* qa, int M, int H, int dim, int rot, int rot_dims,
                          int kv_rank, float eps, lia_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LIA_B200_H_ */
