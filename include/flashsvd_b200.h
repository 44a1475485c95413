/* flashsvd_b200 — C ABI of the B200 decode path for SVD-factored (W = U·V) Llama-shaped models.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (as void*), enqueues
 * work on that stream without synchronising, and returns an int status:
 *     0  ok
 *    <0  argument / shape / alignment / launch error (text via fsvd_last_error_string())
 * Device-side waits are bounded; if one runs out, a non-zero word is left in the workspace and
 * is returned by fsvd_workspace_status() / fsvd_model_status().  The word is sticky until it is
 * cleared (fsvd_workspace_clear_status / fsvd_workspace_init / fsvd_model_reset_sync); the launch
 * that set it still ends by itself and later launches on the same workspace work normally.
 *
 * Launches that share one workspace (or one model) must be ordered one after another on the
 * device (one stream, or events): the workspace holds the vectors the stages hand to each other.
 *
 * Factor naming follows the reference: for a projection d_in -> r -> d_out the input-side
 * factor is `*_v` with nn.Linear weight layout [r, d_in] and the output-side factor is `*_u`
 * with layout [d_out, r]; y = u(v(x)).  All matrices are row-major and contiguous, element type
 * given by `dtype`.  "Reference" paths below are relative to the FlashSVD repository root.
 */
#ifndef FLASHSVD_B200_H_
#define FLASHSVD_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FSVD_DTYPE_BF16 0 /* bf16 storage, fp32 accumulation, outputs rounded to bf16 */
#define FSVD_DTYPE_F32 1  /* fp32 storage and arithmetic (greedy-parity mode) */
#define FSVD_DTYPE_BF16_Q4 2 /* as FSVD_DTYPE_BF16, but every U and V factor pointer is an int4-g128
                                tile stream made by fsvd_q4_pack (norm weights, embedding, lm_head,
                                caches, rope tables and activations stay bf16).  Accepted by
                                fsvd_lowrank_proj, fsvd_lift, fsvd_mlp_swiglu_decode,
                                fsvd_qkv_rope_append, fsvd_decode_layer and fsvd_model_create. */

#define FSVD_OK 0
#define FSVD_ERR_ARG (-1)
#define FSVD_ERR_UNSUPPORTED (-2)
#define FSVD_ERR_ALIGN (-3)
#define FSVD_ERR_WORKSPACE (-4)
#define FSVD_ERR_CUDA (-5)
#define FSVD_ERR_DEVICE_WAIT (-6)
#define FSVD_ERR_CACHE_FULL (-7)

/* Shapes of one model / layer.  Ranks must be multiples of 8, d and I multiples of 8,
 * Dh in {64, 128}, H/Hk in {1, 2, 4, 8}.  Batch: B <= 8 (bf16, int4) / 4 (fp32) runs in the
 * persistent single-launch kernel; 9 <= B <= 128 (bf16 only, gate and up ranks equal) runs as
 * tiled tensor-core GEMMs (tcgen05, accumulators in tensor memory) + batched attention, several
 * launches per layer, accepted by fsvd_workspace_bytes, fsvd_decode_layer and fsvd_model_*.
 * Those three entry points also take the tiled path for bf16 batches of 5..8 (it is faster from 5
 * sequences on; FSVD_TILE_MIN_BATCH moves the threshold, 9 = never); the per-op entry points always
 * use the single-launch kernel. */
typedef struct fsvd_dims {
  int dtype;
  int B;       /* independent sequences */
  int d;       /* hidden size */
  int H, Hk;   /* query heads, key/value heads */
  int Dh;      /* head dim */
  int I;       /* SwiGLU intermediate size */
  int Rq, Rk, Rv, Ro; /* attention ranks */
  int Rg, Ru, Rd;     /* gate / up / down ranks */
  int S_max;   /* cache capacity in tokens */
  int vocab;
  int n_layers;
  float eps;   /* RMSNorm epsilon */
  int rows_are_positions; /* 0: the B rows are independent sequences with cache rows 0..B-1.
                             1: the B rows are consecutive positions of ONE sequence (a chunk of
                             its prompt): every row reads and writes cache row 0, row b at position
                             cache_seqlens[b] (the caller sets cache_seqlens[b] = first + b), and
                             attends positions <= its own, i.e. causally over the chunk.  Accepted
                             by fsvd_decode_layer and fsvd_model_create; the caches are then
                             [1, S_max, Hk, Dh].  The reference fills the cache with its prefill
                             kernels (kernels/flashsvdropeattn.py:67-427) + cache.update
                             (runtime/cache/attn_dense_kv.py:138-191). */
} fsvd_dims;

/* Device pointers of one decoder layer. */
typedef struct fsvd_layer {
  const void* ln1_w;    /* [d]            input_layernorm.weight */
  const void* qkv_v;    /* [Rq+Rk+Rv, d]  cat(q_v_proj, k_v_proj, v_v_proj).weight */
  const void* q_u;      /* [H*Dh, Rq] */
  const void* k_u;      /* [Hk*Dh, Rk] */
  const void* v_u;      /* [Hk*Dh, Rv] */
  const void* o_v;      /* [Ro, H*Dh] */
  const void* o_u;      /* [d, Ro] */
  const void* ln2_w;    /* [d]            post_attention_layernorm.weight */
  const void* upgate_v; /* [Ru+Rg, d]     cat(up_v_proj, gate_v_proj).weight — up rows first,
                           the PCat order of kernels/mlp/decode/dual_split_triton_pcat_s.py:81-90 */
  const void* gate_u;   /* [I, Rg] */
  const void* up_u;     /* [I, Ru] */
  const void* down_v;   /* [Rd, I] */
  const void* down_u;   /* [d, Rd] */
  void* k_cache;        /* [B, S_max, Hk, Dh] keys after RoPE (runtime/cache/attn_dense_kv.py:7-15) */
  void* v_cache;        /* [B, S_max, Hk, Dh] */
} fsvd_layer;

typedef struct fsvd_model fsvd_model;

/* ---- library ---------------------------------------------------------------------------- */
int fsvd_version(void);
const char* fsvd_last_error_string(void);
/* SM count and opt-in shared memory per block of the current device. */
int fsvd_device_props(int* sm_count, int* smem_optin_bytes);
/* Launch geometry.  warps: 0 or 7 (the kernel runs 7 consumer warps + 1 TMA producer warp per
 * CTA); depth: slots of the shared-memory ring of 7 KB boxes (0 = as many as fit, at most
 * 21; rounded down to a multiple of 7); grid: number of CTAs (0 = one per SM).  Defaults come
 * from FSVD_SLOTS / FSVD_GRID or (0, 0).  The grid may be changed between launches on the same
 * workspace: every launch counts its grid barriers from zero.  A model keeps the geometry it
 * was created with. */
int fsvd_set_launch_config(int warps, int depth, int grid);
/* Budget of every device-side wait (at the grid barrier, for a ring box) in SM clocks; default
 * 4e9 (about 2 s) or FSVD_WAIT_CLOCKS; at least 1000.  A wait that runs out sets the status word,
 * and the CTA goes through the rest of the launch without waiting again.  The reference has no
 * counterpart (its kernels do not wait for each other). */
int fsvd_set_wait_limit(long long sm_clocks);

/* Stage timeline for profiling (the analogue of the reference's per-module CUDA-event hooks,
 * utils/evaluator.py:553-689).  While a device buffer of at least nstages * grid * 128 bytes is
 * set, every launch records for each (stage, CTA) sixteen 8-byte slots of %globaltimer values:
 * 0 stage entry, 1 grid barrier passed, 2 input vector staged, 3 stage done, 4 vector loaded,
 * 5 norm reduced, 7 factor boxes consumed, 8 plans made, 10 CTA synchronised, 11 epilogue done.
 * NULL switches it off. */
int fsvd_set_trace_buffer(void* dev_ptr, size_t bytes);

/* ---- workspace -------------------------------------------------------------------------- */
/* Scratch (global memory beyond inputs and outputs) for the per-op entry points and
 * fsvd_decode_layer; zero it once with fsvd_workspace_init before first use. */
size_t fsvd_workspace_bytes(const fsvd_dims* dims);
int fsvd_workspace_init(void* ws, size_t ws_bytes, void* stream);
/* Blocking: copies the device status word back.  0 = nothing happened; 1 / 2 = a wait at the
 * grid barrier / for a ring box ran out (FSVD_ERR_DEVICE_WAIT, the message names the stage);
 * 4 = a token arrived at a cache position >= S_max and its key / value were dropped
 * (FSVD_ERR_CACHE_FULL; the reference raises IndexError there,
 * runtime/cache/attn_dense_kv.py:295-298).  The first event wins. */
int fsvd_workspace_status(void* ws, int* device_status);
/* Clears the status word on `stream` (the rest of the workspace is left as it is). */
int fsvd_workspace_clear_status(void* ws, void* stream);
/* Self-test of the bounded waits: launches a one-stage program whose stage stands behind a grid
 * barrier that nothing arrives at.  The launch ends by itself after the wait budget
 * (fsvd_set_wait_limit) and leaves status 1 with stage index 0; the workspace stays usable (the
 * barrier count is back at zero).  Nothing faults or hangs. */
int fsvd_selftest_wait_timeout(void* ws, size_t ws_bytes, void* stream);

/* ---- per-op entry points ------------------------------------------------------------------
 * y[B,d_out] = (residual +) u(v(x)).  Replaces the two F.linear GEMVs of the low-rank output
 * projection o_u_proj(o_v_proj(a)) (reference: utils/model_utils.py:640 for the shapes,
 * benchmark/attn/bench_real_checkpoint_decode_reconstruct.py:116-123 for y = u(v(x))). */
int fsvd_lowrank_proj(const void* x, const void* v, const void* u, const void* residual, void* y,
                      int B, int d_in, int R, int d_out, int dtype,
                      void* ws, size_t ws_bytes, void* stream);

/* y[B,d_out] = (residual +) p[B,R] @ u[d_out,R]^T: one factor, no rank step.  Replaces the
 * vendor matmuls of reconstruct_qkv_token_shared_prepacked, Q = Pq @ Vq_flat
 * (reference: kernels/attn/decode/densekv_reconstruct_triton.py:693-760), with u = Vq_flat^T =
 * the q_u_proj weight as stored. */
int fsvd_lift(const void* p, const void* u, const void* residual, void* y, int B, int R, int d_out,
              int dtype, void* ws, size_t ws_bytes, void* stream);

/* The same projection for callers that cannot hand over a workspace.  This entry point has no
 * counterpart in the reference.  Its scratch (sync words + rank-space partial sums) is a
 * fixed 256 KiB + 256 B array inside the library's device image, so the call performs no device
 * memory allocation or release of any kind (no cudaMalloc / cudaFree, no memory pool, no
 * allocating library call); on the host it uses ordinary heap for the stage list, and the first
 * time a given set of arguments is seen, for the cached copy of the finished program.  Meant for code that runs where device allocation is off limits
 * or unaffordable: a serving loop whose memory is fully budgeted up front, a real-time thread that
 * must not take the allocator's locks, or a plug-in that is handed tensors but no allocator.
 *  - Limit: B * R <= 8192 (for example B = 1 with R up to 8192, or B = 8 with R up to 1024);
 *    beyond that the call returns FSVD_ERR_WORKSPACE and launches nothing.
 *  - The first call on each device looks up the array's device address and clears its sync
 *    words on `stream`; make that first call during start-up, outside any stream capture and
 *    with the target device current.  Later calls do no set-up.
 *  - One array per device is shared by every call: calls must be ordered one after another
 *    (same stream, or events between streams).  Two calls that overlap in time race on the
 *    partial sums and give undefined results.
 *  - fsvd_static_status reads (and optionally resets) the status word of the array.
 * Both entry points build their stages with the same routine (same K segments, same summation
 * order), so the results are bitwise identical to fsvd_lowrank_proj with the same launch
 * configuration. */
int fsvd_lowrank_proj_static(const void* x, const void* v, const void* u, const void* residual,
                             void* y, int B, int d_in, int R, int d_out, int dtype, void* stream);
/* Blocking (synchronises the device): status word of the built-in scratch of the current device
 * (see fsvd_workspace_status for the codes and the return value); reset != 0 also zeroes the
 * status and the barrier words.  Allocates nothing. */
int fsvd_static_status(int* device_status, int reset);

/* y[B,d] = (residual +) down_u(down_v(silu(gate_u(p_gate)) * up_u(p_up))).
 * With upgate_v != NULL: x is the hidden state [B,d], optionally RMS-normalised by norm_w, and
 * [p_up | p_gate] = upgate_v(x).  With upgate_v == NULL: x is PCat [B, Ru+Rg] = [p_up | p_gate],
 * the input of flashsvd_mlp_dual_split_triton_pcat_s
 * (kernels/mlp/decode/dual_split_triton_pcat_s.py:123-218, kernel :39-120); gate_u/up_u/down_v/
 * down_u here are the nn.Linear weights, i.e. the transposes of that function's GateU/UpU/DownV/
 * DownU arguments. */
int fsvd_mlp_swiglu_decode(const void* x, const void* norm_w, float eps, const void* upgate_v,
                           const void* gate_u, const void* up_u, const void* down_v,
                           const void* down_u, const void* residual, void* y,
                           int B, int d, int I, int Ru, int Rg, int Rd, int dtype,
                           void* ws, size_t ws_bytes, void* stream);

/* Current-token q/k/v from rank space with RoPE and cache append, one launch.  Replaces the
 * packed rank projection hidden @ packed_qkv_rank
 * (benchmark/attn/bench_real_checkpoint_decode_reconstruct.py:125-127), the lift
 * reconstruct_qkv_token_shared{,_hetero,_prepacked}
 * (kernels/attn/decode/densekv_reconstruct_triton.py:464-760) and the rotary + cache-append half
 * of flash_attn_with_kvcache (runtime/attn/decode_registry.py:177-211).  q_out[B,H,Dh] is the
 * rotated query; k (rotated) and v are written at position cache_seqlens[b] of the caches.
 * cos/sin are [S_max, Dh/2] tables of type dtype (runtime/cache/attn_dense_kv.py:331-357). */
int fsvd_qkv_rope_append(const void* x, const void* norm_w, float eps, const void* qkv_v,
                         const void* q_u, const void* k_u, const void* v_u,
                         const void* cos_tab, const void* sin_tab, void* k_cache, void* v_cache,
                         const int* cache_seqlens, void* q_out,
                         int B, int d, int H, int Hk, int Dh, int Rq, int Rk, int Rv, int S_max,
                         int dtype, void* ws, size_t ws_bytes, void* stream);

/* out[B,H,Dh] = softmax(q·K^T * scale)·V over the first cache_seqlens[b] + seqlen_add cached
 * positions (GQA by head grouping), split over the keys and combined in split order.  Replaces
 * the attention half of flash_attn_with_kvcache (runtime/attn/decode_registry.py:177-211);
 * scale <= 0 selects 1/sqrt(Dh). */
int fsvd_flash_decode(const void* q, const void* k_cache, const void* v_cache,
                      const int* cache_seqlens, int seqlen_add, void* out,
                      int B, int H, int Hk, int Dh, int S_max, float scale, int dtype,
                      void* ws, size_t ws_bytes, void* stream);

/* One whole decoder layer for one new token per sequence, one launch:
 * x_out = h + mlp(rms(h)), h = x_in + attn(rms(x_in)); the layer's caches receive the new
 * token at position cache_seqlens[b].  Replaces transformers' LlamaDecoderLayer.forward as the
 * reference drives it from utils/evaluator.py:69-78 in mode="flashsvd". */
int fsvd_decode_layer(const fsvd_dims* dims, const fsvd_layer* layer, const void* cos_tab,
                      const void* sin_tab, const int* cache_seqlens, const void* x_in, void* x_out,
                      void* ws, size_t ws_bytes, void* stream);

/* ---- whole-model decode -------------------------------------------------------------------
 * A model owns a device-resident stage program and its scratch (allocated here, once).  One
 * step = embed -> n_layers decoder layers -> final RMSNorm -> lm_head -> argmax in ONE launch;
 * token ids and sequence lengths live on the device, so consecutive steps need no host
 * round-trip (the reference builds torch.tensor([pos]) and calls .item() every token,
 * scripts/demo_support/api.py:285-312, utils/evaluator.py:39-82,505-512). */
int fsvd_model_create(const fsvd_dims* dims, const fsvd_layer* layers, const void* embed,
                      const void* final_norm_w, const void* lm_head, const void* cos_tab,
                      const void* sin_tab, int max_steps, fsvd_model** out);
int fsvd_model_destroy(fsvd_model* m);
/* Enqueue n_steps greedy decode steps: one kernel launch per step for B <= 8, one CUDA graph launch
 * per step (captured by fsvd_model_create) for B > 8. */
int fsvd_model_step(fsvd_model* m, int n_steps, void* stream);
/* Device buffers: tokens[B] (in: token to feed, out: sampled token), seqlens[B],
 * token_log[max_steps,B], step_counter[1], logits[B,vocab] fp32; `hidden` is the library's internal
 * hidden-state buffer between layers ([B,d] in the model dtype), exposed for debugging. */
int fsvd_model_buffers(fsvd_model* m, int** tokens, int** seqlens, int** token_log,
                       int** step_counter, float** logits, float** hidden);
/* Number of stages of the model's program (sizes the trace buffer); for B > 8 the number of
 * kernel launches of a step. */
int fsvd_model_num_stages(fsvd_model* m);
/* Grid barriers per launch of the model's program (one in front of every stage that reads what
 * the stage before it wrote: 9 per layer + 2). */
int fsvd_model_num_barriers(fsvd_model* m);
/* Blocking: as fsvd_workspace_status, for the model's own scratch. */
int fsvd_model_status(fsvd_model* m, int* device_status);
/* Clears the status, the barrier words and the attention arrival counters after an error. */
int fsvd_model_reset_sync(fsvd_model* m, void* stream);
/* int4 factors: src/quant/packed_quant_linear.py:18-35 (format), :126-171 (pack_weight), :285-300
 * (dequantize: w = scale * (q - zero), groups of 128 along the input dimension).  The reference
 * keeps a dense dequantised copy for decode; here the codes are multiplied as they stream in
 * (y = sum over groups of scale * sum_k (q - 8) x_k, fp32 accumulation) and nothing dense is made.
 * fsvd_q4_pack copies one PackedQuantLinear ([rows, K]: qweight uint8 [rows, K/2] with the low
 * nibble = even input index, scales fp16 [rows, ceil(K/128)], zeros int16 [rows, ceil(K/128)] or
 * NULL) into a stream of fsvd_q4_packed_bytes(rows, K) bytes that the kernels read with TMA: tiles
 * of 16 rows x 1024 inputs, each 16 x 512 bytes of codes (nibbles regrouped inside every 32-bit word: even inputs in the
 * low half-word, odd inputs in the high one) followed by 512 bytes holding the tile's
 * 16 x 8 scales.  Only the symmetric format is supported: with zeros != NULL the call
 * synchronises the stream and returns FSVD_ERR_UNSUPPORTED when a zero point differs from 8.
 * K must be a multiple of 8.  A matrix made by concatenating factors along rows (qkv_v, upgate_v,
 * [q_u; k_u; v_u]) is packed after concatenation, or part by part at byte offsets
 * fsvd_q4_packed_bytes(rows_before, K) when rows_before is a multiple of 16. */
size_t fsvd_q4_packed_bytes(int rows, int K);
int fsvd_q4_pack(const void* qweight, const void* scales, const void* zeros, int rows, int K,
                 void* out, void* stream);

/* ---- Tensor-parallel decode: one model over the GPUs of a node, one process per GPU ----------
 * No counterpart in the reference (it has no multi-GPU decode path; it places whole layers on
 * devices, runtime/cache/attn_dense_kv.py:52-58).  Partitioning: each of `world` ranks holds H / world
 * query heads with their Hk / world key / value heads and I / world columns of the SwiGLU
 * intermediate: q_u, k_u, v_u, gate_u, up_u sharded by rows, o_v and down_v by columns, the other
 * factors replicated; fsvd_dims carries the rank's H, Hk and I.  The partial sums [B, d] of the
 * output projection and of the down projection are exchanged inside the kernels: the epilogue of
 * the GEMM that produces them stores every finished tile straight into an exchange region of every
 * rank (peer stores over NVLink) and raises a flag per CTA; the kernel that follows polls the flags
 * of its own region, adds the `world` partial sums in rank order plus the residual, and applies the
 * next RMSNorm.  No collective library call is on the path.  Waits for a peer are bounded by
 * fsvd_set_wait_limit; when one runs out the workspace status reads 8 (FSVD_ERR_DEVICE_WAIT) and the
 * step completes with whatever arrived.
 *
 * Set-up per rank: allocate a region (fsvd_exchange_region_alloc, zero-filled), export it
 * (fsvd_exchange_region_export: 64 opaque bytes to send to the other processes by any means),
 * import the other ranks' regions (fsvd_exchange_region_import), and create the exchange from the
 * `world` base pointers in rank order (regions[rank] = the rank's own).  All ranks must have
 * allocated before any rank runs a layer.  Every rank must run the same sequence of
 * fsvd_tp_decode_layer calls on one exchange. */
typedef struct fsvd_exchange fsvd_exchange;
size_t fsvd_exchange_region_bytes(int world, int max_rows, int d);
int fsvd_exchange_region_alloc(size_t bytes, void** region);
int fsvd_exchange_region_free(void* region);
int fsvd_exchange_region_export(void* region, unsigned char handle[64]);
int fsvd_exchange_region_import(const unsigned char handle[64], void** region);
int fsvd_exchange_region_release(void* imported_region);
int fsvd_exchange_create(int rank, int world, void* const* regions, int max_rows, int d, void* stream,
                         fsvd_exchange** out);
int fsvd_exchange_destroy(fsvd_exchange* ex);
/* Timing of the exchanges for profiling: while a device buffer is set, the reduction of exchange
 * number k writes record k mod (bytes / 24) = three %globaltimer values (ns): its dependency met
 * (the rank's own GEMM has finished), all ranks' flags seen, reduction done.  Set it before the
 * first layer call that should be traced; NULL switches it off. */
int fsvd_exchange_set_trace(fsvd_exchange* ex, void* dev_ptr, size_t bytes);
/* One decoder layer on this rank's shards (bf16, 1 <= B <= max_rows rows, tiled tensor-core path
 * at every batch size): x_out = the full layer output, identical on every rank.  The workspace has
 * fsvd_tp_workspace_bytes(dims) bytes, zeroed once.  The appended key / value rows are the rank's
 * own heads.  Optional, to save the RMSNorm launches between layers: x_norm_in (non-NULL) = the
 * caller already holds ln1-normalised x_in [B, d] (written by the layer before); next_norm_w
 * (non-NULL) = also write rmsnorm(x_out) * next_norm_w to x_norm_out [B, d] (the next layer's ln1,
 * or the model's final norm). */
size_t fsvd_tp_workspace_bytes(const fsvd_dims* dims);
int fsvd_tp_decode_layer(const fsvd_dims* dims, const fsvd_layer* layer, const void* cos_tab,
                         const void* sin_tab, const int* cache_seqlens, const void* x_in,
                         const void* x_norm_in, void* x_out, const void* next_norm_w, void* x_norm_out,
                         fsvd_exchange* ex, void* ws, size_t ws_bytes, void* stream);

/* Kernel launches enqueued by this library since load (for launch accounting). */
long long fsvd_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* FLASHSVD_B200_H_ */
