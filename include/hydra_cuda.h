/*
 * hydra_cuda.h — C ABI of HydraCUDA, the Blackwell (sm_100a) attention + KV-cache backend for Hydra.
 *
 * This is the whole boundary between Hydra's layer runners and the CUDA kernels: plain C, plain
 * pointers and sizes, no C++ or framework types.  Each entry point replaces one method of the
 * kernel protocol that the reference's Metal backend exposes to its runners; the comment above
 * each one cites that method (path within the Hydra repository : line).
 *
 * Conventions
 *   - Every call returns an hc_status.  Nothing aborts or traps; hc_last_error_string() gives the
 *     message of the last failure on the calling thread.
 *   - Device work is enqueued on the caller's stream (a cudaStream_t passed as void*; NULL is the
 *     default stream) and is asynchronous, like encoding into a Metal command buffer.  Stream order
 *     gives the write-then-read guarantee the runners rely on ("append, then attend").
 *   - One caller thread per context.  No call on the step path allocates device memory: the KV
 *     cache and the split-attention workspace are sized once at hc_kv_cache_create.
 *   - Activations (q, k, v, gate, out) are device buffers of `io_dtype` (fp32, as the reference's
 *     buffers are, or bf16).  The cache is bf16.  Sinks and norm weights are bf16 device pointers
 *     read in place, as the reference reads them from the mapped checkpoint.  RoPE tables are fp32.
 *   - Shapes: q/out/gate [tokens][q_heads][head_dim]; k/v [tokens][kv_heads][head_dim].
 *     head_dim must be a multiple of 8 and at most 512 (the reference's own bound,
 *     Sources/HydraMetal/Shaders/attention.metal:115); q_heads / kv_heads must be a power of two
 *     no larger than 16.
 */
#ifndef HYDRA_CUDA_H
#define HYDRA_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HC_API __attribute__((visibility("default")))

/* Replaces the Swift error enums KernelError (Sources/HydraMetal/AttentionKernels.swift:20-32),
 * KVCache.CacheError (Sources/HydraMetal/KVCache.swift:106-122) and MetalContext.ContextError
 * (Sources/HydraMetal/MetalContext.swift:21-42). */
typedef enum hc_status {
    HC_OK = 0,
    HC_ALLOC_FAILED = 1,     /* CacheError.allocationFailed / KernelError.allocationFailed        */
    HC_KV_OVERFLOW = 2,      /* CacheError.overflow                                               */
    HC_DIM_MISMATCH = 3,     /* KernelError.dimensionMismatch, the headDim <= 512 precondition     */
    HC_UNSUPPORTED = 4,      /* CacheError.unsupportedPattern, or a shape no kernel here serves    */
    HC_BAD_REWIND = 5,       /* the precondition of KVCache.rewind(to:)                            */
    HC_CUDA_ERROR = 6,       /* ContextError.commandBufferFailed                                   */
    HC_COMM_ERROR = 7,       /* a sharded call was given inconsistent rank data                    */
    HC_TIMEOUT = 8,          /* a bounded device-side wait gave up (see hc_context_check)          */
    HC_INVALID_ARGUMENT = 9  /* null pointer, negative size, unknown enum value                    */
} hc_status;

typedef enum hc_dtype { HC_F32 = 0, HC_BF16 = 1 } hc_dtype;

/* How a layer's rows are stored (Sources/HydraMetal/KVCache.swift:160-167). */
typedef enum hc_storage {
    HC_STORAGE_AUTO = 0,   /* the reference's rule: ring iff windowed and context > 8192          */
    HC_STORAGE_LINEAR = 1,
    HC_STORAGE_RING = 2
} hc_storage;

/* Which kernel family serves attention.  AUTO is what production runs.  The other values exist so
 * that a measurement can alternate arms inside one process, as the reference's
 * HYDRA_NO_SPLIT_ATTENTION toggle does (Sources/HydraMetal/ForwardEncoder.swift:1007-1016). */
typedef enum hc_kernel_path {
    HC_PATH_AUTO = 0,
    HC_PATH_SIMT = 1,      /* CUDA-core kernels: any head_dim <= 512                                */
    HC_PATH_TENSOR = 2     /* tcgen05 / TMEM / TMA kernels: head_dim 64, 128 or 256                 */
} hc_kernel_path;

typedef enum hc_gate_layout {
    HC_GATE_NONE = 0,
    HC_GATE_SEPARATE = 1,    /* gate is its own [tokens][q_heads][head_dim] buffer                 */
    HC_GATE_INTERLEAVED = 2  /* q is q_proj's raw output [tokens][q_heads][2*head_dim]: head h's
                                query then head h's gate (Sources/HydraMetal/Shaders/qwen.metal:188-204) */
} hc_gate_layout;

typedef struct hc_context hc_context;
typedef struct hc_kv_cache hc_kv_cache;
typedef struct hc_rope_table hc_rope_table;

/* One layer's geometry.  Replaces ModelDescriptor.attentionGeometry(atLayer:) +
 * attentionPattern(atLayer:) as KVCache.init consumes them (Sources/HydraMetal/KVCache.swift:139-157).
 * kv_heads == 0 marks a recurrent layer: it keeps an index and no memory (KVCache.swift:148-156). */
typedef struct hc_layer_desc {
    int q_heads;
    int kv_heads;
    int head_dim;
    int window;      /* 0 = full causal; else the sliding window in tokens                         */
    int storage;     /* hc_storage                                                                 */
} hc_layer_desc;

/* How a cache is split across GPUs.  The reference has no counterpart (single device).
 *   world == 1: no sharding.
 *   HC_SHARD_HEADS:    the caller gives this rank kv_heads/world heads in hc_layer_desc and the
 *                      matching query heads; nothing is exchanged inside attention.
 *   HC_SHARD_SEQUENCE: key tiles of 128 positions are dealt round-robin, tile j to rank j % world.
 *                      Each rank appends only the rows it owns, attends over them, and the ranks'
 *                      partial results are combined by hc_attention_combine (or all in one call:
 *                      hc_attention_decode_sharded).  The entry points that write a finished
 *                      output refuse such a cache with HC_UNSUPPORTED: they would normalise over
 *                      this rank's keys alone. */
typedef enum hc_shard_mode { HC_SHARD_NONE = 0, HC_SHARD_HEADS = 1, HC_SHARD_SEQUENCE = 2 } hc_shard_mode;
typedef struct hc_shard_desc {
    int mode;   /* hc_shard_mode */
    int rank;
    int world;
} hc_shard_desc;

/* Everything one attention call needs besides the buffers.  Replaces the scalar arguments of
 * ForwardEncoder.attention / attentionPrefill / rmsNormHeads / applyRoPE
 * (Sources/HydraMetal/ForwardEncoder.swift:1107-1115, 590-599, 535-538, 974-979). */
typedef struct hc_attn_params {
    int q_heads;
    int kv_heads;
    int head_dim;
    int window;              /* 0 = full causal (must agree with the cache layer's window)         */
    float sm_scale;          /* 1/sqrt(d) for GPT-OSS and Qwen, 1.0 for Gemma                       */
    int io_dtype;            /* hc_dtype of q, k, v, gate, out                                      */
    const void* sinks;       /* bf16 [q_heads] device, or NULL: no sink (the reference passes
                                bf16(-1e30), Sources/HydraMetal/Gemma4LayerRunner.swift:43-49)      */
    /* Per-head RMSNorm before the rotation (Sources/HydraMetal/Shaders/gemma.metal:785-821). */
    int norm_q;              /* 0 = none, 1 = with q_norm_weight, 2 = weightless                    */
    int norm_k;              /* same with k_norm_weight                                             */
    int norm_v;              /* 0 = none, 2 = weightless (Gemma's v_norm)                           */
    const void* q_norm_weight; /* bf16 [head_dim] device                                           */
    const void* k_norm_weight; /* bf16 [head_dim] device                                           */
    float norm_eps;
    /* Rotation of q and k (Sources/HydraMetal/Shaders/attention.metal:48-72).  NULL = none. */
    const hc_rope_table* rope;
    /* Sigmoid output gate (Sources/HydraMetal/Shaders/qwen.metal:211-219). */
    int gate_layout;         /* hc_gate_layout                                                      */
    const void* gate;        /* device, io_dtype, for HC_GATE_SEPARATE                              */
    int kernel_path;         /* hc_kernel_path                                                      */
    /* Bidirectional blocks (an image's tokens see each other), the `blocks` buffer of
     * attention_prefill (Sources/HydraMetal/Shaders/batch.metal:322-324, 340-352; `blockEnds` of
     * BatchEncoder.attention, Sources/HydraMetal/BatchEncoder.swift:210-217).  Device memory, one entry
     * per token of the call: the position one past the end of the block the token belongs to, or 0
     * for an ordinary token; NULL = none.  A token at position p then sees [start, max(p + 1,
     * block end)) with `start` still bounded by the window.  Prefill calls only (decode ignores it).
     * The call is worked in chunks of at most the cache's prefill_chunk tokens and a block reaches no
     * further than the end of its token's chunk, the last key appended by then (the reference reads
     * on, into rows not yet written, when a chunk boundary cuts an image).  The tensor-core kernels
     * take the buffer (head_dim 64, 128, 256: whole rows per item, every item reaching to the chunk's
     * last key tile), the general kernel the rest.  Rows outside the blocks keep, bit for bit, the
     * results of the call without the buffer, and so still equal their decode steps. */
    const int* block_ends;
} hc_attn_params;

/* ---- context -------------------------------------------------------------------------------- */

/* Replaces MetalContext.init (Sources/HydraMetal/MetalContext.swift:44-70): binds a device and
 * checks that it can run these kernels (compute capability 10.x). */
HC_API hc_status hc_context_create(int device, hc_context** out);
HC_API void hc_context_destroy(hc_context* ctx);

/* Replaces the check in MetalContext.wait (Sources/HydraMetal/MetalContext.swift:191-202):
 * synchronises `stream`, then reports a CUDA error or a device-side status word (HC_TIMEOUT if a
 * bounded wait inside a kernel gave up) recorded since the last check. */
HC_API hc_status hc_context_check(hc_context* ctx, void* stream);

/* Message of the last failure on this thread; never NULL. */
HC_API const char* hc_last_error_string(void);

/* Number of kernels this library has launched through `ctx` since it was created (what
 * ForwardEncoder.dispatchCounter counts, Sources/HydraMetal/ForwardEncoder.swift:38-68). */
HC_API uint64_t hc_context_launch_count(const hc_context* ctx);

/* ---- RoPE tables ---------------------------------------------------------------------------- */

/* Replaces RoPETables.write (Sources/HydraCore/RoPETables.swift:98-107) for every position at
 * once: cos(p * f_i) * concentration and sin(...) computed on the host in double, cast to fp32 and
 * uploaded as [positions][pairs].  `inv_freq` has head_dim/2 entries; a zero entry is an unrotated
 * pair (partial rotary).  Prefill and decode read the same table, so they rotate identically. */
HC_API hc_status hc_rope_table_create(hc_context* ctx, const double* inv_freq, int pairs,
                                      double concentration, int positions, hc_rope_table** out);
HC_API void hc_rope_table_destroy(hc_rope_table* table);
/* Device pointers of the table rows (fp32 [positions][pairs]). */
HC_API hc_status hc_rope_table_pointers(const hc_rope_table* table, const float** cos_out,
                                        const float** sin_out, int* positions, int* pairs);

/* Inverse frequencies with the YaRN extension; scaling <= 1 gives plain theta^(-2i/d).
 * Replaces RoPETables.init (Sources/HydraCore/RoPETables.swift:54-85).  Host only. */
HC_API hc_status hc_yarn_inverse_frequencies(int head_dim, double base, int initial_context,
                                             double scaling, double ntk_alpha, double ntk_beta,
                                             double* inv_freq, double* concentration);
/* Plain frequencies with a zero tail.  Replaces Gemma4RoPETables.init
 * (Sources/HydraCore/RoPETables.swift:135-148).  Host only. */
HC_API hc_status hc_inverse_frequencies(int head_dim, double theta, int rotating_pairs,
                                        double* inv_freq);

/* ---- Projections -------------------------------------------------------------------------- */

/* y[t][o] = sum_i x[t][i] * w[o][i] (+ bias[o]): the Q, K, V and O projections on either side of
 * the attention calls, on the tensor cores (tcgen05, fp32 accumulate).  Replaces
 * ForwardEncoder.denseProjection (Sources/HydraMetal/ForwardEncoder.swift:160-190) and
 * BatchEncoder.denseProjection (Sources/HydraMetal/BatchEncoder.swift:104), i.e. bf16_gemv and its
 * batched and tiled forms (Sources/HydraMetal/Shaders/dense.metal:14-60, batch.metal:36-88,
 * tiled.metal:48-120); the weight keeps the reference's layout.
 *   x     bf16 [tokens][in_features]      (the reference passes fp32 activations; round them to bf16)
 *   w     bf16 [out_features][in_features], row-major
 *   bias      bf16 [out_features] or NULL
 *   residual  fp32 [tokens][out_features] added to the result, or NULL; it may be y itself, which
 *             is the layer's `hidden += o_proj(attention)` (Sources/HydraReference/ReferenceLayer.swift:186-187)
 *   y         fp32 or bf16 [tokens][out_features], per y_dtype (fp32 with a residual)
 * in_features must be a multiple of 64; x, w and y 16-byte aligned.  For Qwen's 2x-tall q_proj pass
 * the whole weight: y is then the interleaved query/gate buffer that HC_GATE_INTERLEAVED reads. */
HC_API hc_status hc_linear(hc_context* ctx, const void* x, const void* w, const void* bias,
                           const void* residual, void* y, int tokens, int in_features,
                           int out_features, int y_dtype, void* stream);

/* Up to four projections of the same x in ONE launch (a layer's q_proj, k_proj and v_proj): w, bias,
 * y and out_features are arrays of n entries (bias may be NULL, or hold NULLs).  The results are bit
 * for bit those of n hc_linear calls; what it saves is launches, which is most of a decode-sized
 * call, and the idle SMs of the narrow k and v projections in a prompt-sized one. */
HC_API hc_status hc_linear_group(hc_context* ctx, const void* x, int n, const void* const* w,
                                 const void* const* bias, void* const* y, const int* out_features,
                                 int tokens, int in_features, int y_dtype, void* stream);

/* y = x * rsqrt(mean(x^2) + eps) * scale over whole rows: the layer's input norm.  Replaces
 * ForwardEncoder.rmsNorm (Sources/HydraMetal/ForwardEncoder.swift:141-157) and the batched kernel
 * (Sources/HydraMetal/Shaders/batch.metal:184-218).  x fp32 or bf16 [tokens][width], scale bf16
 * [width] or NULL (rmsNormUnscaled), y fp32 or bf16: bf16 is what hc_linear takes. */
HC_API hc_status hc_rms_norm(hc_context* ctx, const void* x, const void* scale_bf16, void* y,
                             int tokens, int width, float eps, int x_dtype, int y_dtype, void* stream);

/* ---- KV cache ------------------------------------------------------------------------------- */

/* Replaces KVCache.init(model:contextLength:device:) (Sources/HydraMetal/KVCache.swift:132-182).
 * Allocates, per layer, K and V as bf16 [max_seqs][kv_heads][capacity][head_dim] (head-major, so
 * one head's history is contiguous), zero-filled, plus the split-attention workspace.
 * `prefill_chunk` is KVCache.prefillChunk (512 in the reference): a ring reports, and bounds chunks
 * and rewinds by, window + prefill_chunk rows rounded up to a multiple of 128; it is stored one such
 * margin longer (hc_layer_info.capacity), which lets hc_prefill_chunks overlap consecutive chunks.
 * `shard` may be NULL.
 *
 * The call also fixes how each layer groups its 128-key tiles into segments (1024 or 4096 keys),
 * from the layer's head counts, prefill_chunk, max_seqs and the device's SM count: the attention
 * kernels fold tiles into segment partials and segment partials into rows, and a launch may spread
 * a row's segments over thread blocks.  All calls on one cache agree bit for bit (chunked prefill,
 * one-shot prefill, token-by-token decode, any batch); two caches of different geometry may differ
 * in the last bits. */
HC_API hc_status hc_kv_cache_create(hc_context* ctx, const hc_layer_desc* layers, int n_layers,
                                    int context_length, int prefill_chunk, int max_seqs,
                                    const hc_shard_desc* shard, hc_kv_cache** out);
/* The same cache with PAGED storage for its linear (full-attention) layers: instead of
 * context_length rows per sequence, each such layer is one pool of `total_pages` pages of 128 rows
 * (one key tile) shared by all max_seqs sequences, so a ragged batch costs the sum of its lengths
 * rather than max_seqs times the longest.  A page is assigned when a position of its tile is first
 * appended (by whichever layer gets there first: one page table serves all layers), and given back
 * by hc_kv_reset and hc_kv_rewind; an append that finds no free page fails with HC_KV_OVERFLOW.
 * Every other call is unchanged, and results are bit for bit those of the contiguous cache.  Ring
 * layers keep their own rows per sequence.  The reference has no counterpart: its batches share one
 * contiguous cache per slot (Sources/HydraMetal/KVCache.swift:132-182).  total_pages = 0 is
 * hc_kv_cache_create.  Not for sequence-sharded caches. */
HC_API hc_status hc_kv_cache_create_paged(hc_context* ctx, const hc_layer_desc* layers, int n_layers,
                                          int context_length, int prefill_chunk, int max_seqs,
                                          int total_pages, const hc_shard_desc* shard,
                                          hc_kv_cache** out);
/* Free pages of a paged cache, -1 for a contiguous one. */
HC_API int hc_kv_free_pages(const hc_kv_cache* cache);
HC_API void hc_kv_cache_destroy(hc_kv_cache* cache);

/* Replaces KVCache.byteCount (KVCache.swift:184-187): bytes of K and V actually allocated. */
HC_API size_t hc_kv_cache_bytes(const hc_kv_cache* cache);

/* Replaces KVCache.Layer's fields (KVCache.swift:41-66). */
typedef struct hc_layer_info {
    void* keys;          /* device, bf16 */
    void* values;
    int ring_size;       /* 0 for linear storage */
    int capacity;        /* rows per (sequence, head) */
    int entry_bytes;     /* bytes one token occupies in keys (or values): kv_heads * head_dim * 2 */
    int windowed;
    int keeps_history;
} hc_layer_info;
HC_API hc_status hc_kv_layer_info(const hc_kv_cache* cache, int layer, hc_layer_info* out);

/* Copies `tokens` rows starting at `position` of one sequence back to the host, in the reference's
 * row layout [tokens][kv_heads][head_dim] (bf16 bits), synchronously.  For validation: the reference
 * keeps its cache in CPU-visible storage for the same purpose (KVCache.swift:170-172).  On a
 * sequence-sharded cache, rows this rank does not own come back as zeros. */
HC_API hc_status hc_kv_read(hc_context* ctx, const hc_kv_cache* cache, int layer, int seq,
                            int position, int tokens, uint16_t* keys_out, uint16_t* values_out);

/* Sequence sharding arithmetic (host only, no counterpart in the reference): the rank that owns
 * `position` in a world of `world` ranks, and the row it occupies in that rank's storage. */
HC_API int hc_shard_owner(int world, int position);
HC_API int hc_shard_local_row(int world, int position);

/* Replaces KVCache.visibleRange(layer:position:) (KVCache.swift:193-200). */
HC_API hc_status hc_kv_visible_range(const hc_kv_cache* cache, int layer, int position, int* start,
                                     int* count);
/* Replace KVCache.length / advance() / reset() / rewindFloor / canRewind(to:) / rewind(to:)
 * (KVCache.swift:68, 202-213, 215-217, 95-104, 223-229), per sequence. */
HC_API hc_status hc_kv_length(const hc_kv_cache* cache, int seq, int* length);
HC_API hc_status hc_kv_advance(hc_kv_cache* cache, int seq, int tokens);
HC_API hc_status hc_kv_reset(hc_kv_cache* cache, int seq);
HC_API hc_status hc_kv_rewind_floor(const hc_kv_cache* cache, int seq, int* floor);
HC_API int hc_kv_can_rewind(const hc_kv_cache* cache, int seq, int tokens);
HC_API hc_status hc_kv_rewind(hc_kv_cache* cache, int seq, int tokens);

/* ---- the kernel protocol -------------------------------------------------------------------- */

/* Replaces ForwardEncoder.writeKeyValue (Sources/HydraMetal/ForwardEncoder.swift:989-1005, one
 * token) and BatchEncoder.writeKeyValue (Sources/HydraMetal/BatchEncoder.swift:190-208, a chunk):
 * token t of k, v goes to position first_position + t (modulo the ring).  When params asks for it,
 * the per-head norm of k (and weightless norm of v) and the rotation of k are applied first, in
 * that order, fused into the same kernel; with norm_k = norm_v = 0 and rope = NULL this is the
 * reference's plain cast-and-store.  Does not move the sequence length: call hc_kv_advance. */
HC_API hc_status hc_kv_append(hc_context* ctx, hc_kv_cache* cache, int layer, int seq,
                              const void* k, const void* v, int tokens, int first_position,
                              const hc_attn_params* params, void* stream);

/* The same for one token of each of n_seq sequences (a batched decode step): row i of k, v goes to
 * sequence seq_ids[i] at positions[i].  seq_ids and positions are HOST arrays.  The reference runs
 * one sequence at a time and has no counterpart. */
HC_API hc_status hc_kv_append_batch(hc_context* ctx, hc_kv_cache* cache, int layer,
                                    const int* seq_ids, const int* positions, int n_seq,
                                    const void* k, const void* v, const hc_attn_params* params,
                                    void* stream);

/* Replaces BatchEncoder.attention (Sources/HydraMetal/BatchEncoder.swift:210-246) and
 * ForwardEncoder.attentionPrefill (Sources/HydraMetal/ForwardEncoder.swift:590-631): causal
 * attention of `tokens` queries at positions first_position .. first_position + tokens - 1 over
 * the cache (the chunk's own keys must have been appended first).  The q norm and rotation asked
 * for in params are applied to q first; the sigmoid gate is applied last.  Image blocks
 * (blockEnds) are not supported: text only. */
HC_API hc_status hc_attention_prefill(hc_context* ctx, hc_kv_cache* cache, int layer, int seq,
                                      const void* q, void* out, int tokens, int first_position,
                                      const hc_attn_params* params, void* stream);

/* Replaces ForwardEncoder.attention (Sources/HydraMetal/ForwardEncoder.swift:1107-1165) together
 * with the split kernel and its merge (ForwardEncoder.swift:1064-1105,
 * Sources/HydraMetal/Shaders/attention.metal:307-452): one query token per sequence.
 * seq_ids and positions are HOST arrays of n_seq entries (n_seq = 1 is the reference's case);
 * q and out are [n_seq][q_heads][head_dim].  positions[i] is the query's own position: its key
 * must already be in the cache.  The visible range follows hc_kv_visible_range. */
HC_API hc_status hc_attention_decode(hc_context* ctx, hc_kv_cache* cache, int layer,
                                     const int* seq_ids, const int* positions, int n_seq,
                                     const void* q, void* out, const hc_attn_params* params,
                                     void* stream);

/* hc_attention_decode for callers that cannot allocate device memory.  It has no counterpart in the
 * reference, whose split partials come from a scratch pool grown on demand
 * (Sources/HydraMetal/MetalContext.swift:108-116).
 *
 * Who needs it: a runner that has already given every free byte of the device to its weight and KV
 * pools, a plugin that must not touch its host process's allocator, or code running where
 * cudaMalloc is not allowed.  The split-decode partials of this call live in one fixed array
 * inside the library (hc_attention_decode_static_limit() bytes, 8 MiB, held by every GPU that
 * loads the library until the process exits) and the call performs no cudaMalloc, cudaFree or any
 * other allocating routine.
 *
 *   - q must be bf16, already normalised and rotated: io_dtype HC_BF16, norm_q 0, rope NULL, gate
 *     none or HC_GATE_SEPARATE.  1 to 64 sequences; not for sequence-sharded caches.
 *   - A call whose partials (n_seq * q_heads * slots * (head_dim + 2) floats, where slots is the
 *     number of segments of 1024 or 4096 keys, or of 128-key tiles, that the library cuts the longest
 *     sequence into for this batch) exceed the limit is refused with HC_KV_OVERFLOW and a message
 *     that states both sizes.
 *   - It runs the same kernels as hc_attention_decode (tcgen05 for head_dim 64, 128, 256, CUDA
 *     cores otherwise, params->kernel_path honoured) with the partials redirected, so its output
 *     equals hc_attention_decode's bit for bit.
 *   - The array's device address is looked up by hc_context_create (cudaGetSymbolAddress, with the
 *     context's device current), which also makes the CUDA runtime load the module that holds the
 *     array: the 8 MiB are reserved when the context is created, not inside a later call.  Create
 *     the context before starting a stream capture and before handing the device's memory away.
 *   - All calls share the array and it keeps the last call's contents.  Nothing in it needs to be
 *     zero beforehand: each call writes every partial before reading it.  Two calls that overlap on
 *     the GPU (different streams, no dependency) race on it: serialise them. */
HC_API size_t hc_attention_decode_static_limit(void);
HC_API hc_status hc_attention_decode_static(hc_context* ctx, hc_kv_cache* cache, int layer,
                                            const int* seq_ids, const int* positions, int n_seq,
                                            const void* q, void* out, const hc_attn_params* params,
                                            void* stream);

/* Sequence-sharded attention, step 1 of 2 (no counterpart in the reference).  Like
 * hc_attention_prefill / hc_attention_decode over the key tiles this rank owns, but writes this
 * rank's unnormalised partial (running maximum, denominator, numerator) instead of the output:
 * fp32 [rows][q_heads][head_dim + 2] with rows = tokens (prefill) or n_seq (decode), laid out as
 * head_dim numerators, then the maximum, then the denominator.  The sink is counted by rank 0
 * only.  The caller all-gathers the ranks' partials (NCCL) into [world][rows][q_heads][head_dim+2]
 * and every rank calls hc_attention_combine on the gathered buffer. */
HC_API size_t hc_attention_partial_bytes(const hc_attn_params* params, int rows);
HC_API hc_status hc_attention_prefill_partial(hc_context* ctx, hc_kv_cache* cache, int layer,
                                              int seq, const void* q, void* partial, int tokens,
                                              int first_position, const hc_attn_params* params,
                                              void* stream);
HC_API hc_status hc_attention_decode_partial(hc_context* ctx, hc_kv_cache* cache, int layer,
                                             const int* seq_ids, const int* positions, int n_seq,
                                             const void* q, void* partial,
                                             const hc_attn_params* params, void* stream);
/* Step 2 of 2: folds the `world` partials in rank order (the same log-sum-exp merge as
 * Sources/HydraMetal/Shaders/attention.metal:418-452), divides, applies the gate, writes `out`.
 * Every rank computes the same bits.  `q` is only read for HC_GATE_INTERLEAVED (the gate sits
 * beside the query); pass NULL otherwise. */
HC_API hc_status hc_attention_combine(hc_context* ctx, const void* gathered, int world, int rows,
                                      const void* q, void* out, const hc_attn_params* params,
                                      void* stream);

/* ---- shards: the same two steps as one call, the exchange inside the library ------------------ */

/* This rank's place among the GPUs that share a model (no counterpart in the reference).
 * `nccl_comm` is an ncclComm_t the caller initialised (ncclCommInitRank) and keeps alive; it is
 * needed for HC_SHARD_SEQUENCE over more than one rank and for hc_linear_sharded (head shards
 * exchange nothing inside attention and may pass NULL if they do not call it), and its size and
 * rank must agree with `world` and `rank`: a mismatch, like any
 * inconsistent (mode, rank, world), is HC_COMM_ERROR.  `max_partial_bytes` is the largest
 * hc_attention_partial_bytes(params, rows) a sharded call will need; the exchange buffers
 * ((world + 1) times that) are allocated here, not on the step path. */
typedef struct hc_shard hc_shard;
HC_API hc_status hc_shard_create(hc_context* ctx, void* nccl_comm, int mode, int rank, int world,
                                 size_t max_partial_bytes, hc_shard** out);
HC_API void hc_shard_destroy(hc_shard* shard);
/* The hc_shard_desc to create this rank's cache with. */
HC_API hc_status hc_shard_describe(const hc_shard* shard, hc_shard_desc* desc);

/* hc_attention_decode / hc_attention_prefill on a sharded cache, complete: for a sequence shard
 * this rank's partial, ncclAllGather of the ranks' partials into this GPU's memory and the combine
 * are enqueued on `stream` in that order, and every rank ends with the same bits in `out`.  For a
 * head shard (or a world of one) they are the plain calls.  The cache must have been created with
 * hc_shard_describe's description. */
HC_API hc_status hc_attention_decode_sharded(hc_context* ctx, hc_shard* shard, hc_kv_cache* cache,
                                             int layer, const int* seq_ids, const int* positions,
                                             int n_seq, const void* q, void* out,
                                             const hc_attn_params* params, void* stream);
HC_API hc_status hc_attention_prefill_sharded(hc_context* ctx, hc_shard* shard, hc_kv_cache* cache,
                                              int layer, int seq, const void* q, void* out,
                                              int tokens, int first_position,
                                              const hc_attn_params* params, void* stream);

/* The output projection of a head-sharded layer (row-parallel o_proj).  x is this rank's attention
 * output, bf16 [tokens][in_features] with in_features = its own heads x head_dim; w the matching
 * columns of W_o held as a matrix of its own, bf16 [out_features][in_features]; y fp32
 * [tokens][out_features] on every rank.  Each rank's hc_linear gives its partial sums into y (rank
 * 0's with the bias and the residual, which may be y itself), then NCCL adds them on `stream` through
 * the communicator the shard was created with (any hc_shard_mode):
 *   scatter = 0  ncclAllReduce in place: every rank ends with the whole y, the same bits on all;
 *   scatter = 1  ncclReduceScatter in place: rank r ends with rows [r * tokens / world, (r + 1) *
 *                tokens / world) of y summed (tokens must divide); its other rows hold partials.
 * A world of one is hc_linear.  The collective is NCCL's own kernel after the GEMM, not fused with
 * it.  No counterpart in the reference, which runs on one device. */
HC_API hc_status hc_linear_sharded(hc_context* ctx, hc_shard* shard, const void* x, const void* w,
                                   const void* bias, const void* residual, void* y, int tokens,
                                   int in_features, int out_features, int scatter, void* stream);


/* Stand-alone forms of the element-wise kernels, for runners that call them one by one as the
 * reference does.  In place on `vector` (io_dtype).
 * hc_rms_norm_heads replaces ForwardEncoder.rmsNormHeads (ForwardEncoder.swift:535-551) and
 * BatchEncoder.rmsNormHeadsBatch (BatchEncoder.swift:429-446); weight NULL = weightless.
 * hc_apply_rope replaces ForwardEncoder.applyRoPE / applyRoPEBatched (ForwardEncoder.swift:974-987,
 * 702-719) and BatchEncoder.applyRoPE (BatchEncoder.swift:175-188): token t uses the table row of
 * position first_position + t. */
HC_API hc_status hc_rms_norm_heads(hc_context* ctx, void* vector, const void* weight_bf16,
                                   int tokens, int heads, int head_dim, float eps, int io_dtype,
                                   void* stream);
HC_API hc_status hc_apply_rope(hc_context* ctx, void* vector, const hc_rope_table* table,
                               int tokens, int heads, int head_dim, int first_position,
                               int io_dtype, void* stream);
/* Replaces ForwardEncoder.qwenSplitQueryGate (ForwardEncoder.swift:856-869). */
HC_API hc_status hc_qwen_split_query_gate(hc_context* ctx, const void* combined, void* query,
                                          void* gate, int tokens, int heads, int head_dim,
                                          int io_dtype, void* stream);
/* Replaces ForwardEncoder.qwenApplyOutputGate (ForwardEncoder.swift:872-882). */
HC_API hc_status hc_qwen_apply_output_gate(hc_context* ctx, void* output, const void* gate,
                                           size_t count, int io_dtype, void* stream);

/* ---- one layer's step ------------------------------------------------------------------------- */

/* Append + attend for `tokens` tokens of one sequence in one call, DEVICE buffers: the per-layer
 * order of the reference's encoders (norm -> RoPE -> cache write -> attention -> gate:
 * Sources/HydraMetal/ForwardEncoder.swift attention block; Sources/HydraReference/
 * Gemma4ReferenceLayer.swift:154-157, 234-246) as one entry point.  Results are bit for bit those
 * of hc_kv_append followed by hc_attention_prefill (tokens > 1) or hc_attention_decode
 * (tokens == 1); for a chunk that fits the prologue workspace the K/V append and the query prologue
 * share one launch.  It does not move the sequence length. */
HC_API hc_status hc_layer_step(hc_context* ctx, hc_kv_cache* cache, int layer, int seq,
                               const void* q, const void* k, const void* v, void* out, int tokens,
                               int first_position, const hc_attn_params* params, void* stream);

/* hc_layer_step for a whole prompt: `tokens` tokens in chunks of `chunk` (the reference's
 * PrefillRunner loop, Sources/HydraMetal/PrefillRunner.swift:128-184, one call per prompt instead of
 * one per chunk).  Each chunk is one hc_layer_step and the results are bit for bit those of the
 * chunk-by-chunk calls.  The work starts behind whatever `stream` holds at the call and `stream` ends
 * behind all of it, like any other call; in between, on layers with linear storage, the library
 * runs a chunk's prologue one chunk ahead and alternate chunks' attention on two streams of its
 * own (ordered by events), so that a chunk's kernels start while the previous chunk's are still
 * finishing. */
HC_API hc_status hc_prefill_chunks(hc_context* ctx, hc_kv_cache* cache, int layer, int seq,
                                   const void* q, const void* k, const void* v, void* out,
                                   int tokens, int first_position, int chunk,
                                   const hc_attn_params* params, void* stream);

/* ---- host-buffer convenience (what a runner without device buffers of its own calls) --------- */

/* One whole step of the path with HOST buffers: copies q, k, v (and gate) to the device, appends,
 * attends (prefill if tokens > 1, decode otherwise), copies `out` back and synchronises the stream.
 * It does not move the sequence length (a model calls it once per layer and hc_kv_advance once per
 * token).  The copies go through a device staging buffer owned by the cache; they are part of the
 * call, which takes at most max(prefill_chunk, max_seqs) tokens.  q/k/v/gate/out are host pointers of params->io_dtype; params->gate must be a HOST
 * pointer here.  Replaces nothing one-to-one: on Apple Silicon the reference's buffers are shared
 * between CPU and GPU (Sources/HydraMetal/KVCache.swift:170-172), so its runners never copy. */
HC_API hc_status hc_layer_step_host(hc_context* ctx, hc_kv_cache* cache, int layer, int seq,
                                    const void* q, const void* k, const void* v, void* out,
                                    int tokens, int first_position, const hc_attn_params* params,
                                    void* stream);

/* The same for a whole prompt in chunks of `chunk` tokens (at most max(prefill_chunk, max_seqs)): the
 * copy in of chunk i + 1 and the copy out of chunk i - 1 run under the kernels of chunk i (two
 * staging slots, the library's own copy streams, events), and the call returns when every result is
 * on the host.  Use pinned host memory, or the copies serialise. */
HC_API hc_status hc_prefill_host(hc_context* ctx, hc_kv_cache* cache, int layer, int seq,
                                 const void* q, const void* k, const void* v, void* out,
                                 int tokens, int first_position, int chunk,
                                 const hc_attn_params* params, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HYDRA_CUDA_H */
