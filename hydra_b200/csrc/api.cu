// api.cu — the C ABI declared in include/hydra_cuda.h: argument checking, the KV-cache object and
// its bookkeeping, and the choice of kernels for each call.  All device work is in the other files.

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "internal.hpp"

namespace hc {

static thread_local std::string g_last_error = "";

hc_status fail(hc_status status, const std::string& message) {
    g_last_error = message;
    return status;
}

hc_status check_cuda(cudaError_t err, const char* what) {
    if (err == cudaSuccess) return HC_OK;
    return fail(HC_CUDA_ERROR, std::string(what) + ": " + cudaGetErrorString(err));
}

namespace {

int round_up(int value, int multiple) { return (value + multiple - 1) / multiple * multiple; }

size_t dtype_bytes(int dtype) { return dtype == HC_F32 ? 4 : 2; }

// KVCache.linearWindowLimit (Sources/HydraMetal/KVCache.swift:130).
constexpr int kLinearWindowLimit = 8192;

bool group_ok(int group) { return group == 1 || group == 2 || group == 4 || group == 8 || group == 16; }

hc_status validate_params(const hc_kv_cache* cache, int layer, const hc_attn_params* p) {
    if (!cache || !p) return fail(HC_INVALID_ARGUMENT, "null cache or params");
    if (layer < 0 || layer >= int(cache->layers.size())) return fail(HC_INVALID_ARGUMENT, "layer index out of range");
    const hc_layer_store& L = cache->layers[size_t(layer)];
    if (!L.keeps_history) {
        return fail(HC_UNSUPPORTED, "layer " + std::to_string(layer) + " keeps a recurrent state, not a key/value history");
    }
    if (p->head_dim != L.desc.head_dim || p->kv_heads != L.desc.kv_heads) {
        return fail(HC_DIM_MISMATCH, "params geometry differs from the cache layer's");
    }
    if (p->q_heads <= 0 || p->q_heads > L.desc.q_heads || p->q_heads % p->kv_heads != 0 ||
        !group_ok(p->q_heads / p->kv_heads)) {
        return fail(HC_DIM_MISMATCH, "q_heads must be a power-of-two multiple (<= 16) of kv_heads and no larger than the layer's");
    }
    if (p->window != L.desc.window) return fail(HC_DIM_MISMATCH, "params.window differs from the cache layer's window");
    if (p->io_dtype != HC_F32 && p->io_dtype != HC_BF16) return fail(HC_INVALID_ARGUMENT, "unknown io_dtype");
    if (p->norm_q == 1 && !p->q_norm_weight) return fail(HC_INVALID_ARGUMENT, "norm_q = 1 without q_norm_weight");
    if (p->norm_k == 1 && !p->k_norm_weight) return fail(HC_INVALID_ARGUMENT, "norm_k = 1 without k_norm_weight");
    if (p->norm_v == 1) return fail(HC_INVALID_ARGUMENT, "norm_v takes 0 or 2 (weightless): v_norm has no weight");
    if (p->rope && p->rope->pairs != p->head_dim / 2) return fail(HC_DIM_MISMATCH, "rope table pairs != head_dim / 2");
    if (p->gate_layout == HC_GATE_SEPARATE && !p->gate) return fail(HC_INVALID_ARGUMENT, "HC_GATE_SEPARATE without a gate buffer");
    if (p->gate_layout < HC_GATE_NONE || p->gate_layout > HC_GATE_INTERLEAVED) return fail(HC_INVALID_ARGUMENT, "unknown gate_layout");
    if (!(p->sm_scale > 0.0f)) return fail(HC_INVALID_ARGUMENT, "sm_scale must be positive");
    return HC_OK;
}

CacheView view_of(const hc_kv_cache* cache, const hc_layer_store& L) {
    CacheView view;
    view.k = L.k;
    view.v = L.v;
    view.capacity = L.capacity;
    view.kv_heads = L.desc.kv_heads;
    view.map.ring = L.ring;
    const bool sequence = cache->shard.mode == HC_SHARD_SEQUENCE && cache->shard.world > 1;
    view.map.rank = sequence ? cache->shard.rank : 0;
    view.map.world = sequence ? cache->shard.world : 1;
    view.map.log_segment = L.log_segment;
    const bool paged = cache->pages_dev != nullptr && L.ring == 0;
    view.map.pages = paged ? cache->pages_dev : nullptr;
    view.map.pages_per_seq = paged ? cache->pages_per_seq : 0;
    return view;
}

AttnShape shape_of(const hc_kv_cache* cache, const hc_attn_params* p, bool partial_mode) {
    AttnShape shape;
    shape.q_heads = p->q_heads;
    shape.kv_heads = p->kv_heads;
    shape.head_dim = p->head_dim;
    shape.group = p->q_heads / p->kv_heads;
    shape.window = p->window;
    shape.c = p->sm_scale * kLog2e;
    shape.sinks = static_cast<const uint16_t*>(p->sinks);
    const bool sequence = cache->shard.mode == HC_SHARD_SEQUENCE && cache->shard.world > 1;
    shape.count_sink = (partial_mode && sequence && cache->shard.rank != 0) ? 0 : 1;
    return shape;
}

// A sequence-sharded cache holds only this rank's key tiles: an entry point that writes a finished
// output from it would normalise over a fraction of the keys, silently.  Only the partial forms,
// whose results hc_attention_combine folds over the ranks, may read it.
hc_status check_shard_mode(const hc_kv_cache* cache, bool partial_mode) {
    if (!partial_mode && cache->shard.mode == HC_SHARD_SEQUENCE && cache->shard.world > 1) {
        return fail(HC_UNSUPPORTED, "this cache is sequence-sharded over " + std::to_string(cache->shard.world) +
                                        " ranks: use the _partial entry points and hc_attention_combine");
    }
    return HC_OK;
}

bool needs_q_prepare(const hc_attn_params* p) {
    return p->io_dtype != HC_BF16 || p->norm_q != 0 || p->rope != nullptr ||
           p->gate_layout == HC_GATE_INTERLEAVED;
}

// Rows a position range needs; checks capacity the way KVCache.advance does (KVCache.swift:202-213).
hc_status check_positions(const hc_kv_cache* cache, const hc_layer_store& L, int first, int tokens,
                          const hc_attn_params* p) {
    if (tokens < 0 || first < 0) return fail(HC_INVALID_ARGUMENT, "negative token count or position");
    if (L.ring == 0 && first + tokens > cache->context_length) {
        return fail(HC_KV_OVERFLOW, "position " + std::to_string(first + tokens - 1) + " beyond capacity " +
                                        std::to_string(cache->context_length));
    }
    if (L.ring > 0 && tokens > L.ring_margin) {
        return fail(HC_KV_OVERFLOW, "a chunk of " + std::to_string(tokens) + " tokens overruns the ring's margin of " +
                                        std::to_string(L.ring_margin));
    }
    if (p->rope && first + tokens > p->rope->positions) {
        return fail(HC_DIM_MISMATCH, "rope table is shorter than the positions asked for");
    }
    return HC_OK;
}

void fill_q_job(PrepJob& job, const hc_attn_params* p, const void* q, void* dst) {
    const int d = p->head_dim;
    const int mult = p->gate_layout == HC_GATE_INTERLEAVED ? 2 : 1;
    job.src = q;
    job.src_dtype = p->io_dtype;
    job.heads = p->q_heads;
    job.token_stride = (long long)p->q_heads * d * mult;
    job.head_stride = d * mult;
    job.norm = p->norm_q;
    job.weight = static_cast<const uint16_t*>(p->q_norm_weight);
    job.rope = p->rope ? 1 : 0;
    job.kind = 0;
    job.dst = dst;
}

void fill_kv_jobs(PrepArgs& args, int at, const hc_attn_params* p, const void* k, const void* v) {
    const int d = p->head_dim;
    PrepJob& jk = args.job[at];
    jk.src = k;
    jk.src_dtype = p->io_dtype;
    jk.heads = p->kv_heads;
    jk.token_stride = (long long)p->kv_heads * d;
    jk.head_stride = d;
    jk.norm = p->norm_k;
    jk.weight = static_cast<const uint16_t*>(p->k_norm_weight);
    jk.rope = p->rope ? 1 : 0;
    jk.kind = 1;
    jk.dst = nullptr;
    PrepJob& jv = args.job[at + 1];
    jv = jk;
    jv.src = v;
    jv.norm = p->norm_v;
    jv.weight = nullptr;
    jv.rope = 0;
    jv.kind = 2;
}

void fill_common(PrepArgs& args, const hc_attn_params* p) {
    args.head_dim = p->head_dim;
    args.eps = p->norm_eps;
    args.cos = p->rope ? p->rope->cos : nullptr;
    args.sin = p->rope ? p->rope->sin : nullptr;
    args.table_positions = p->rope ? p->rope->positions : 0;
}

const unsigned char* offset_rows(const void* base, size_t rows, size_t row_elems, int dtype) {
    return static_cast<const unsigned char*>(base) + rows * row_elems * dtype_bytes(dtype);
}

bool use_tensor_path(const hc_attn_params* p, const AttnShape& shape, hc_status* status) {
    *status = HC_OK;
    const char* env = std::getenv("HYDRA_CUDA_FORCE_SIMT");
    if (p->kernel_path == HC_PATH_SIMT || (p->kernel_path == HC_PATH_AUTO && env && env[0] == '1')) return false;
    const bool ok = tc_supported(shape);
    if (p->kernel_path == HC_PATH_TENSOR && !ok) {
        *status = fail(HC_UNSUPPORTED, "the tcgen05 path serves head_dim 64, 128 and 256 only");
        return false;
    }
    return ok;
}

// The body shared by hc_attention_prefill and hc_attention_prefill_partial.
// With k_fused / v_fused set (hc_layer_step; one pass, tokens <= the prologue workspace) the K/V
// append of the same tokens rides in the Q prologue's launch.
// Paged storage: every 128-key tile of [first, first + tokens) of `seq` gets a page (all layers share
// the table, so whichever layer appends a position first assigns it), and the new entries are copied
// to the device table on `stream`, ahead of the kernel that writes the rows.
hc_status ensure_pages(hc_kv_cache* cache, const hc_layer_store& L, int seq, int first, int tokens, cudaStream_t stream) {
    if (!cache->pages_dev || L.ring != 0 || tokens <= 0) return HC_OK;
    int* table = cache->pages_host + size_t(seq) * cache->pages_per_seq;
    int lo = -1, hi = -1;
    for (int tile = first / kTileKeys; tile <= (first + tokens - 1) / kTileKeys; ++tile) {
        if (table[tile] >= 0) continue;
        if (cache->free_pages.empty()) {
            return fail(HC_KV_OVERFLOW, "the paged cache is out of pages (" + std::to_string(cache->total_pages) +
                                            " of 128 rows): sequence " + std::to_string(seq) + " needs one for position " +
                                            std::to_string(tile * kTileKeys));
        }
        table[tile] = cache->free_pages.back();
        cache->free_pages.pop_back();
        if (lo < 0) lo = tile;
        hi = tile;
    }
    if (lo < 0) return HC_OK;
    const size_t offset = size_t(seq) * cache->pages_per_seq + lo;
    return check_cuda(cudaMemcpyAsync(cache->pages_dev + offset, cache->pages_host + offset, size_t(hi - lo + 1) * sizeof(int),
                                      cudaMemcpyHostToDevice, stream), "page table update");
}

// Gives back the pages of `seq` from key tile `first_tile` on.
void release_pages(hc_kv_cache* cache, int seq, int first_tile) {
    if (!cache->pages_host) return;
    int* table = cache->pages_host + size_t(seq) * cache->pages_per_seq;
    for (int tile = std::max(first_tile, 0); tile < cache->pages_per_seq; ++tile) {
        if (table[tile] >= 0) {
            cache->free_pages.push_back(table[tile]);
            table[tile] = -1;
        }
    }
}

// When `ahead` is given (hc_prefill_chunks), the prologue launch goes to ahead->stream into the
// ahead->slot-th prepared-query buffer, and `stream` waits for ahead->done, recorded behind it: the
// prologue of a chunk can then run while the previous chunk's attention is still finishing.
struct PrologueAhead {
    cudaStream_t stream;
    cudaEvent_t done;
    int slot;
};

hc_status prefill_impl(hc_context* ctx, hc_kv_cache* cache, int layer, int seq, const void* q,
                       void* out, int tokens, int first_position, const hc_attn_params* p,
                       bool partial_mode, cudaStream_t stream, const void* k_fused = nullptr,
                       const void* v_fused = nullptr, const PrologueAhead* ahead = nullptr) {
    if (!ctx || !q || !out) return fail(HC_INVALID_ARGUMENT, "null context or buffer");
    hc_status st = validate_params(cache, layer, p);
    if (st != HC_OK) return st;
    if (seq < 0 || seq >= cache->max_seqs) return fail(HC_INVALID_ARGUMENT, "sequence index out of range");
    hc_layer_store& L = cache->layers[size_t(layer)];
    st = check_positions(cache, L, first_position, tokens, p);
    if (st != HC_OK) return st;
    if (tokens == 0) return HC_OK;

    st = check_shard_mode(cache, partial_mode);
    if (st != HC_OK) return st;
    const AttnShape shape = shape_of(cache, p, partial_mode);
    const CacheView view = view_of(cache, L);
    const bool tensor = use_tensor_path(p, shape, &st);
    if (st != HC_OK) return st;
    const int d = p->head_dim;
    const int mult = p->gate_layout == HC_GATE_INTERLEAVED ? 2 : 1;
    const bool prep = needs_q_prepare(p);
    int step = prep ? cache->ws.qprep_tokens : tokens;
    // Bidirectional blocks: chunk by chunk (a block ends with its token's chunk).
    const int* blocks = p->block_ends;
    if (blocks) step = std::min(step, cache->prefill_chunk);

    for (int start = 0; start < tokens; start += step) {
        const int count = std::min(step, tokens - start);
        const unsigned char* q_rows = offset_rows(q, size_t(start), size_t(p->q_heads) * d * mult, p->io_dtype);
        const uint16_t* q_bf16 = reinterpret_cast<const uint16_t*>(q_rows);
        if (prep || k_fused) {
            PrepArgs args{};
            fill_common(args, p);
            int jobs = 0;
            if (k_fused) {
                st = ensure_pages(cache, L, seq, first_position + start, count, ahead ? ahead->stream : stream);
                if (st != HC_OK) return st;
            }
            uint16_t* prepared = cache->ws.qprep + (ahead ? size_t(ahead->slot) * cache->ws.qprep_slot_elems : 0);
            if (prep) fill_q_job(args.job[jobs++], p, q_rows, prepared);
            if (k_fused) {
                fill_kv_jobs(args, jobs, p, k_fused, v_fused);
                jobs += 2;
            }
            args.n_jobs = jobs;
            args.tokens = count;
            args.first_position = first_position + start;
            args.batched = 0;
            args.seq = seq;
            args.cache = view;
            st = launch_prepare(ctx, args, ahead ? ahead->stream : stream);
            if (st != HC_OK) return st;
            if (ahead) {
                cudaError_t err = cudaEventRecord(ahead->done, ahead->stream);
                if (err == cudaSuccess) err = cudaStreamWaitEvent(stream, ahead->done, 0);
                if (err != cudaSuccess) return check_cuda(err, "prefill: prologue event");
            }
            if (prep) q_bf16 = prepared;
        }
        EpilogueArgs ep{};
        ep.io_dtype = p->io_dtype;
        ep.write_partial = partial_mode ? 1 : 0;
        ep.gate_layout = partial_mode ? HC_GATE_NONE : p->gate_layout;
        if (partial_mode) {
            ep.out = static_cast<float*>(out) + size_t(start) * p->q_heads * (d + 2);
        } else {
            ep.out = const_cast<unsigned char*>(offset_rows(out, size_t(start), size_t(p->q_heads) * d, p->io_dtype));
        }
        if (ep.gate_layout == HC_GATE_SEPARATE) {
            ep.gate = offset_rows(p->gate, size_t(start), size_t(p->q_heads) * d, p->io_dtype);
        } else if (ep.gate_layout == HC_GATE_INTERLEAVED) {
            ep.gate = q_rows;
        }
        if (tensor) {
            // A chunk attended to on the second stream works in the upper halves of the workspace.
            Workspace ws = cache->ws;
            if (ahead) {
                ws.part_o += size_t(ahead->slot) * ws.prefill_o_floats;
                ws.part_ml += size_t(ahead->slot) * ws.prefill_ml_floats;
                ws.part_o_floats = ws.prefill_o_floats;
                ws.part_ml_floats = ws.prefill_ml_floats;
            }
            st = tc_prefill(ctx, shape, L, view, seq, q_bf16, count, first_position + start, ws, ep, stream,
                            blocks ? blocks + start : nullptr);
        } else {
            st = simt_prefill(ctx, shape, view, seq, q_bf16, count, first_position + start, ep, stream,
                              blocks ? blocks + start : nullptr);
        }
        if (st != HC_OK) return st;
    }
    return HC_OK;
}

// With k_fused / v_fused set (hc_layer_step, one token) the K/V append rides in the Q prologue's launch.
hc_status decode_impl(hc_context* ctx, hc_kv_cache* cache, int layer, const int* seq_ids,
                      const int* positions, int n_seq, const void* q, void* out,
                      const hc_attn_params* p, bool partial_mode, cudaStream_t stream,
                      const void* k_fused = nullptr, const void* v_fused = nullptr) {
    if (!ctx || !q || !out || !seq_ids || !positions) return fail(HC_INVALID_ARGUMENT, "null context or buffer");
    hc_status st = validate_params(cache, layer, p);
    if (st != HC_OK) return st;
    if (n_seq < 0) return fail(HC_INVALID_ARGUMENT, "negative sequence count");
    hc_layer_store& L = cache->layers[size_t(layer)];
    for (int b = 0; b < n_seq; ++b) {
        if (seq_ids[b] < 0 || seq_ids[b] >= cache->max_seqs) return fail(HC_INVALID_ARGUMENT, "sequence index out of range");
        st = check_positions(cache, L, positions[b], 1, p);
        if (st != HC_OK) return st;
    }
    st = check_shard_mode(cache, partial_mode);
    if (st != HC_OK) return st;
    const AttnShape shape = shape_of(cache, p, partial_mode);
    const CacheView view = view_of(cache, L);
    const bool tensor = use_tensor_path(p, shape, &st);
    if (st != HC_OK) return st;
    const int d = p->head_dim;
    const int mult = p->gate_layout == HC_GATE_INTERLEAVED ? 2 : 1;
    const bool prep = needs_q_prepare(p);
    // A launch takes as many sequences as the prepared-query buffer has rows for.
    const int per_launch = prep ? std::min(kMaxBatch, cache->ws.qprep_tokens) : kMaxBatch;

    for (int start = 0; start < n_seq; start += per_launch) {
        const int count = std::min(per_launch, n_seq - start);
        BatchMeta meta{};
        for (int b = 0; b < count; ++b) {
            meta.seq[b] = seq_ids[start + b];
            meta.pos[b] = positions[start + b];
        }
        const unsigned char* q_rows = offset_rows(q, size_t(start), size_t(p->q_heads) * d * mult, p->io_dtype);
        const uint16_t* q_bf16 = reinterpret_cast<const uint16_t*>(q_rows);
        if (prep || k_fused) {
            PrepArgs args{};
            fill_common(args, p);
            int jobs = 0;
            if (prep) fill_q_job(args.job[jobs++], p, q_rows, cache->ws.qprep);
            if (k_fused) {
                for (int b = 0; b < count; ++b) {
                    st = ensure_pages(cache, L, meta.seq[b], meta.pos[b], 1, stream);
                    if (st != HC_OK) return st;
                }
                const size_t kv_row = size_t(p->kv_heads) * d;
                fill_kv_jobs(args, jobs, p, offset_rows(k_fused, size_t(start), kv_row, p->io_dtype),
                             offset_rows(v_fused, size_t(start), kv_row, p->io_dtype));
                jobs += 2;
            }
            args.n_jobs = jobs;
            args.tokens = count;
            args.batched = 1;
            args.meta = meta;
            args.cache = view;
            st = launch_prepare(ctx, args, stream);
            if (st != HC_OK) return st;
            if (prep) q_bf16 = cache->ws.qprep;
        }
        EpilogueArgs ep{};
        ep.io_dtype = p->io_dtype;
        ep.write_partial = partial_mode ? 1 : 0;
        ep.gate_layout = partial_mode ? HC_GATE_NONE : p->gate_layout;
        if (partial_mode) {
            ep.out = static_cast<float*>(out) + size_t(start) * p->q_heads * (d + 2);
        } else {
            ep.out = const_cast<unsigned char*>(offset_rows(out, size_t(start), size_t(p->q_heads) * d, p->io_dtype));
        }
        if (ep.gate_layout == HC_GATE_SEPARATE) {
            ep.gate = offset_rows(p->gate, size_t(start), size_t(p->q_heads) * d, p->io_dtype);
        } else if (ep.gate_layout == HC_GATE_INTERLEAVED) {
            ep.gate = q_rows;
        }
        if (tensor) st = tc_decode(ctx, shape, L, view, meta, count, q_bf16, cache->ws, ep, stream);
        else st = simt_decode(ctx, shape, view, meta, count, q_bf16, cache->ws, ep, stream);
        if (st != HC_OK) return st;
    }
    return HC_OK;
}

}  // namespace

// Argument checking and kernel arguments for hc_attention_decode_static (attn_simt.cu).  Nothing
// here allocates.
hc_status static_decode_inputs(hc_context* ctx, hc_kv_cache* cache, int layer, const int* seq_ids,
                               const int* positions, int n_seq, const void* q, void* out,
                               const hc_attn_params* p, AttnShape* shape, CacheView* view, BatchMeta* meta,
                               EpilogueArgs* ep, const hc_layer_store** store, bool* tensor) {
    if (!ctx || !q || !out || !seq_ids || !positions) return fail(HC_INVALID_ARGUMENT, "null context or buffer");
    hc_status st = validate_params(cache, layer, p);
    if (st != HC_OK) return st;
    if (p->io_dtype != HC_BF16 || p->norm_q != 0 || p->rope != nullptr || p->gate_layout == HC_GATE_INTERLEAVED) {
        return fail(HC_UNSUPPORTED, "hc_attention_decode_static takes a bf16 query that is already normalised and "
                                    "rotated (io_dtype bf16, norm_q 0, rope NULL, gate none or separate)");
    }
    if (n_seq < 1 || n_seq > kMaxBatch) {
        return fail(HC_INVALID_ARGUMENT, "hc_attention_decode_static takes 1 to " + std::to_string(kMaxBatch) + " sequences");
    }
    if (cache->shard.mode == HC_SHARD_SEQUENCE && cache->shard.world > 1) {
        return fail(HC_UNSUPPORTED, "hc_attention_decode_static does not serve a sequence-sharded cache");
    }
    const hc_layer_store& L = cache->layers[size_t(layer)];
    for (int b = 0; b < n_seq; ++b) {
        if (seq_ids[b] < 0 || seq_ids[b] >= cache->max_seqs) return fail(HC_INVALID_ARGUMENT, "sequence index out of range");
        st = check_positions(cache, L, positions[b], 1, p);
        if (st != HC_OK) return st;
        meta->seq[b] = seq_ids[b];
        meta->pos[b] = positions[b];
    }
    *shape = shape_of(cache, p, false);
    *view = view_of(cache, L);
    *store = &L;
    *tensor = use_tensor_path(p, *shape, &st);          // the same choice hc_attention_decode makes
    if (st != HC_OK) return st;
    ep->out = out;
    ep->io_dtype = p->io_dtype;
    ep->write_partial = 0;
    ep->gate_layout = p->gate_layout;
    ep->gate = p->gate;
    return HC_OK;
}

}  // namespace hc

using namespace hc;

extern "C" {

const char* hc_last_error_string(void) { return g_last_error.c_str(); }

hc_status hc_context_create(int device, hc_context** out) {
    if (!out) return fail(HC_INVALID_ARGUMENT, "null out pointer");
    *out = nullptr;
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess || count == 0) {
        return fail(HC_CUDA_ERROR, std::string("no CUDA device: ") + cudaGetErrorString(err));
    }
    if (device < 0 || device >= count) return fail(HC_INVALID_ARGUMENT, "device index out of range");
    cudaDeviceProp prop{};
    err = cudaGetDeviceProperties(&prop, device);
    if (err != cudaSuccess) return check_cuda(err, "cudaGetDeviceProperties");
    if (prop.major != 10) {
        return fail(HC_UNSUPPORTED, "this library holds sm_100a code only; device is compute capability " +
                                        std::to_string(prop.major) + "." + std::to_string(prop.minor));
    }
    err = cudaSetDevice(device);
    if (err != cudaSuccess) return check_cuda(err, "cudaSetDevice");
    hc_context* ctx = new (std::nothrow) hc_context();
    if (!ctx) return fail(HC_ALLOC_FAILED, "out of host memory");
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    err = cudaMalloc(&ctx->status_dev, sizeof(int));
    if (err == cudaSuccess) err = cudaMemset(ctx->status_dev, 0, sizeof(int));
    if (err == cudaSuccess) err = cudaMallocHost(&ctx->status_host, sizeof(int));
    if (err != cudaSuccess) {
        hc_context_destroy(ctx);
        return fail(HC_ALLOC_FAILED, std::string("context status word: ") + cudaGetErrorString(err));
    }
    *ctx->status_host = 0;
    // The fixed scratch of hc_attention_decode_static: its address is looked up here, once, with this
    // device current, which also makes the runtime load that module (and reserve the array) now
    // rather than inside the first call that must not allocate.
    const hc_status scratch = static_scratch_prepare(device, &ctx->static_scratch);
    if (scratch != HC_OK) {
        const std::string message = g_last_error;
        hc_context_destroy(ctx);
        g_last_error = message;
        return scratch;
    }
    *out = ctx;
    return HC_OK;
}

void hc_context_destroy(hc_context* ctx) {
    if (!ctx) return;
    if (ctx->status_dev) cudaFree(ctx->status_dev);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    delete ctx;
}

hc_status hc_context_check(hc_context* ctx, void* stream) {
    if (!ctx) return fail(HC_INVALID_ARGUMENT, "null context");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaMemcpyAsync(ctx->status_host, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    if (err != cudaSuccess) return check_cuda(err, "stream synchronise");
    const int word = *ctx->status_host;
    if (word != 0) {
        cudaMemsetAsync(ctx->status_dev, 0, sizeof(int), s);
        cudaStreamSynchronize(s);
        return fail(HC_TIMEOUT, "a kernel gave up a bounded wait (status word " + std::to_string(word) + ")");
    }
    return HC_OK;
}

uint64_t hc_context_launch_count(const hc_context* ctx) { return ctx ? ctx->launches : 0; }

// ---- RoPE tables --------------------------------------------------------------------------------

hc_status hc_yarn_inverse_frequencies(int head_dim, double base, int initial_context, double scaling,
                                      double ntk_alpha, double ntk_beta, double* inv_freq,
                                      double* concentration) {
    if (!inv_freq || !concentration || head_dim <= 0 || head_dim % 2) return fail(HC_INVALID_ARGUMENT, "bad arguments");
    const int pairs = head_dim / 2;
    if (!(scaling > 1.0)) {
        *concentration = 1.0;
        for (int i = 0; i < pairs; ++i) inv_freq[i] = 1.0 / std::pow(base, double(2 * i) / double(head_dim));
        return HC_OK;
    }
    *concentration = 0.1 * std::log(scaling) + 1.0;
    const double half_dim = double(head_dim) / 2.0;
    const double two_pi = 2.0 * 3.14159265358979323846;
    const double low = half_dim * std::log(double(initial_context) / (ntk_beta * two_pi)) / std::log(base);
    const double high = half_dim * std::log(double(initial_context) / (ntk_alpha * two_pi)) / std::log(base);
    if (!(low > 0 && low < high && high < half_dim - 1)) return fail(HC_INVALID_ARGUMENT, "inconsistent YaRN bounds");
    for (int i = 0; i < pairs; ++i) {
        const double frequency = std::pow(base, double(2 * i) / double(head_dim));
        const double ramp = (double(i) - low) / (high - low);
        const double mask = 1.0 - std::min(std::max(ramp, 0.0), 1.0);
        inv_freq[i] = (1.0 / (scaling * frequency)) * (1.0 - mask) + (1.0 / frequency) * mask;
    }
    return HC_OK;
}

hc_status hc_inverse_frequencies(int head_dim, double theta, int rotating_pairs, double* inv_freq) {
    if (!inv_freq || head_dim <= 0 || head_dim % 2) return fail(HC_INVALID_ARGUMENT, "bad arguments");
    const int pairs = head_dim / 2;
    const int rotating = std::min(std::max(rotating_pairs, 0), pairs);
    for (int i = 0; i < pairs; ++i) {
        inv_freq[i] = i < rotating ? 1.0 / std::pow(theta, 2.0 * double(i) / double(head_dim)) : 0.0;
    }
    return HC_OK;
}

hc_status hc_rope_table_create(hc_context* ctx, const double* inv_freq, int pairs, double concentration,
                               int positions, hc_rope_table** out) {
    if (!ctx || !inv_freq || !out || pairs <= 0 || positions <= 0) return fail(HC_INVALID_ARGUMENT, "bad arguments");
    *out = nullptr;
    const size_t count = size_t(positions) * pairs;
    std::vector<float> host_cos(count), host_sin(count);
    for (int p = 0; p < positions; ++p) {
        const double t = double(p);
        for (int i = 0; i < pairs; ++i) {
            host_cos[size_t(p) * pairs + i] = float(std::cos(t * inv_freq[i]) * concentration);
            host_sin[size_t(p) * pairs + i] = float(std::sin(t * inv_freq[i]) * concentration);
        }
    }
    hc_rope_table* table = new (std::nothrow) hc_rope_table();
    if (!table) return fail(HC_ALLOC_FAILED, "out of host memory");
    table->device = ctx->device;
    table->positions = positions;
    table->pairs = pairs;
    cudaError_t err = cudaSetDevice(ctx->device);
    if (err == cudaSuccess) err = cudaMalloc(&table->cos, count * sizeof(float));
    if (err == cudaSuccess) err = cudaMalloc(&table->sin, count * sizeof(float));
    if (err == cudaSuccess) err = cudaMemcpy(table->cos, host_cos.data(), count * sizeof(float), cudaMemcpyHostToDevice);
    if (err == cudaSuccess) err = cudaMemcpy(table->sin, host_sin.data(), count * sizeof(float), cudaMemcpyHostToDevice);
    if (err != cudaSuccess) {
        hc_rope_table_destroy(table);
        return fail(HC_ALLOC_FAILED, std::string("rope table: ") + cudaGetErrorString(err));
    }
    *out = table;
    return HC_OK;
}

void hc_rope_table_destroy(hc_rope_table* table) {
    if (!table) return;
    if (table->cos) cudaFree(table->cos);
    if (table->sin) cudaFree(table->sin);
    delete table;
}

hc_status hc_rope_table_pointers(const hc_rope_table* table, const float** cos_out, const float** sin_out,
                                 int* positions, int* pairs) {
    if (!table) return fail(HC_INVALID_ARGUMENT, "null table");
    if (cos_out) *cos_out = table->cos;
    if (sin_out) *sin_out = table->sin;
    if (positions) *positions = table->positions;
    if (pairs) *pairs = table->pairs;
    return HC_OK;
}

// ---- KV cache -----------------------------------------------------------------------------------

hc_status hc_kv_cache_create(hc_context* ctx, const hc_layer_desc* layers, int n_layers, int context_length,
                             int prefill_chunk, int max_seqs, const hc_shard_desc* shard, hc_kv_cache** out) {
    return hc_kv_cache_create_paged(ctx, layers, n_layers, context_length, prefill_chunk, max_seqs, 0, shard, out);
}

hc_status hc_kv_cache_create_paged(hc_context* ctx, const hc_layer_desc* layers, int n_layers, int context_length,
                                   int prefill_chunk, int max_seqs, int total_pages, const hc_shard_desc* shard,
                                   hc_kv_cache** out) {
    if (!ctx || !layers || !out || n_layers <= 0 || context_length <= 0 || prefill_chunk <= 0 || max_seqs <= 0 || total_pages < 0) {
        return fail(HC_INVALID_ARGUMENT, "bad arguments to hc_kv_cache_create");
    }
    *out = nullptr;
    hc_shard_desc sd{HC_SHARD_NONE, 0, 1};
    if (shard) {
        sd = *shard;
        if (sd.world < 1 || sd.rank < 0 || sd.rank >= sd.world || sd.mode < HC_SHARD_NONE || sd.mode > HC_SHARD_SEQUENCE) {
            return fail(HC_COMM_ERROR, "inconsistent shard description (mode, rank, world)");
        }
        if (sd.world == 1) sd.mode = HC_SHARD_NONE;
    }
    const bool sequence = sd.mode == HC_SHARD_SEQUENCE;
    if (sequence && total_pages > 0) return fail(HC_UNSUPPORTED, "a paged cache cannot be sequence-sharded");
    cudaError_t err = cudaSetDevice(ctx->device);
    if (err != cudaSuccess) return check_cuda(err, "cudaSetDevice");

    hc_kv_cache* cache = new (std::nothrow) hc_kv_cache();
    if (!cache) return fail(HC_ALLOC_FAILED, "out of host memory");
    cache->ctx = ctx;
    cache->context_length = context_length;
    cache->prefill_chunk = prefill_chunk;
    cache->max_seqs = max_seqs;
    cache->shard = sd;
    cache->lengths.assign(size_t(max_seqs), 0);
    cache->layers.resize(size_t(n_layers));

    size_t max_q_elems = 0, max_kv_elems = 0, part_o_floats = 0, part_ml_floats = 0, prefill_o_floats = 0, prefill_ml_floats = 0;
    hc_status st = HC_OK;
    if (total_pages > 0) {
        cache->total_pages = total_pages;
        cache->pages_per_seq = (context_length + kTileKeys - 1) / kTileKeys;
        const size_t entries = size_t(max_seqs) * cache->pages_per_seq;
        err = cudaMalloc(&cache->pages_dev, entries * sizeof(int));
        if (err == cudaSuccess) err = cudaMemset(cache->pages_dev, 0, entries * sizeof(int));
        if (err == cudaSuccess) err = cudaMallocHost(&cache->pages_host, entries * sizeof(int));
        if (err != cudaSuccess) {
            cudaGetLastError();
            st = fail(HC_ALLOC_FAILED, std::string("page table: ") + cudaGetErrorString(err));
        } else {
            std::fill(cache->pages_host, cache->pages_host + entries, -1);
            cache->free_pages.resize(size_t(total_pages));
            for (int page = 0; page < total_pages; ++page) cache->free_pages[size_t(page)] = total_pages - 1 - page;
        }
    }
    for (int i = 0; i < n_layers && st == HC_OK; ++i) {
        hc_layer_store& L = cache->layers[size_t(i)];
        L.desc = layers[i];
        if (L.desc.kv_heads == 0) {           // recurrent layer: an index and no memory
            L.keeps_history = false;
            continue;
        }
        const int d = L.desc.head_dim;
        if (d <= 0 || d % 8 != 0 || d > 512) {
            st = fail(HC_DIM_MISMATCH, "head_dim " + std::to_string(d) + " must be a multiple of 8 and at most 512");
            break;
        }
        if (L.desc.kv_heads < 0 || L.desc.q_heads <= 0 || L.desc.q_heads % L.desc.kv_heads != 0 ||
            !group_ok(L.desc.q_heads / L.desc.kv_heads) || L.desc.window < 0) {
            st = fail(HC_DIM_MISMATCH, "layer " + std::to_string(i) + ": bad head counts or window");
            break;
        }
        L.keeps_history = true;
        const bool windowed = L.desc.window > 0;
        bool ring = false;
        if (L.desc.storage == HC_STORAGE_AUTO) ring = windowed && context_length > kLinearWindowLimit;
        else if (L.desc.storage == HC_STORAGE_RING) {
            if (!windowed) { st = fail(HC_UNSUPPORTED, "ring storage asked for a full-attention layer"); break; }
            ring = true;
        } else if (L.desc.storage != HC_STORAGE_LINEAR) { st = fail(HC_INVALID_ARGUMENT, "unknown storage"); break; }
        if (ring && sequence) { st = fail(HC_UNSUPPORTED, "ring storage cannot be sequence-sharded"); break; }
        // The reference's ring holds window + prefill_chunk rows (KVCache.swift:160-167; here rounded up
        // to whole tiles): that is what the margin, the reported ring size and the rewind floor
        // follow.  The stored ring is one margin longer, so that the rows a chunk appends never
        // overwrite keys the previous chunk still attends to and hc_prefill_chunks may run a chunk's
        // prologue while the previous chunk's attention is finishing.
        const int reference_ring = ring ? round_up(L.desc.window + prefill_chunk, kTileKeys) : 0;
        L.ring_margin = ring ? reference_ring - L.desc.window : 0;
        L.ring = ring ? round_up(reference_ring + L.ring_margin, kTileKeys) : 0;
        int tiles = (context_length + kTileKeys - 1) / kTileKeys;
        if (sequence) tiles = (tiles + sd.world - 1) / sd.world;
        const bool paged = total_pages > 0 && !ring;
        L.capacity = ring ? L.ring : paged ? total_pages * kTileKeys : tiles * kTileKeys;
        const size_t bytes = size_t(paged ? 1 : max_seqs) * L.desc.kv_heads * L.capacity * d * 2;
        err = cudaMalloc(&L.k, bytes);
        if (err == cudaSuccess) err = cudaMalloc(&L.v, bytes);
        if (err == cudaSuccess) err = cudaMemset(L.k, 0, bytes);
        if (err == cudaSuccess) err = cudaMemset(L.v, 0, bytes);
        if (err != cudaSuccess) {
            cudaGetLastError();
            st = fail(HC_ALLOC_FAILED, "KV cache: cannot allocate " + std::to_string(2 * bytes) + " B for layer " + std::to_string(i));
            break;
        }
        max_q_elems = std::max(max_q_elems, size_t(L.desc.q_heads) * d);
        max_kv_elems = std::max(max_kv_elems, size_t(L.desc.kv_heads) * d);
        // How the layer groups its key tiles (see common.cuh): short segments where launches gain from
        // cutting their rows' keys at little cost in partials, long ones elsewhere.
        //   prefill: when even a full chunk gives too few (row tile, kv head) pairs to occupy the SMs
        //            (half of them; a quarter for head_dim 256, whose kernel pays more per item) and a
        //            row can span more than two short segments;
        //   decode:  a cache for batches of sequences, whose split kernel then leaves one partial per
        //            1024 keys instead of one per 128.
        const int tokens_per_tile = kTileKeys / (L.desc.q_heads / L.desc.kv_heads);
        const int chunk_row_tiles = (prefill_chunk + tokens_per_tile - 1) / tokens_per_tile;
        const int reach = windowed ? std::min(L.desc.window + prefill_chunk, context_length) : context_length;
        const bool few_rows = (d == 256 ? 4 : 2) * chunk_row_tiles * L.desc.kv_heads <= std::max(ctx->sm_count, 1) &&
                              reach > (2 * kTileKeys << kLogSegmentSmall);
        const bool batched = max_seqs >= 8;
        L.log_segment = few_rows || batched ? kLogSegmentSmall : kLogSegmentLarge;
        // Workspace for the partials of split launches.  Decode, at its finest cut: one per (batch
        // entry, query head, key tile of this rank).  Prefill, layers with short segments only: one
        // per (query token, query head, segment).
        const int world = sequence ? sd.world : 1;
        const int decode_reach = windowed ? std::min(L.desc.window + kTileKeys, context_length) : context_length;
        const size_t decode_slots = size_t(((decode_reach + kTileKeys - 1) / kTileKeys + world - 1) / world + 1);
        const size_t decode_rows = size_t(std::min(max_seqs, kMaxBatch)) * L.desc.q_heads;
        part_o_floats = std::max(part_o_floats, decode_rows * decode_slots * d);
        part_ml_floats = std::max(part_ml_floats, decode_rows * decode_slots * 2);
        if (few_rows) {
            const size_t prefill_slots = size_t((((reach + kTileKeys - 1) / kTileKeys) >> kLogSegmentSmall) + 2);
            const size_t prefill_rows = size_t(prefill_chunk) * L.desc.q_heads;
            prefill_o_floats = std::max(prefill_o_floats, prefill_rows * prefill_slots * d);
            prefill_ml_floats = std::max(prefill_ml_floats, prefill_rows * prefill_slots * 2);
        }
        // The tensor-core kernels keep a whole-row launch's second-fold state in the same buffer:
        // head_dim x 128 floats per thread block.
        if (d == 64 || d == 128 || d == 256) prefill_o_floats = std::max(prefill_o_floats, size_t(std::max(ctx->sm_count, 1)) * d * 128);
        st = tc_make_tensor_maps(cache, L);
    }
    if (st == HC_OK && max_q_elems == 0) st = fail(HC_UNSUPPORTED, "no layer keeps a key/value history");
    if (st == HC_OK) {
        hc::Workspace& ws = cache->ws;
        ws.qprep_tokens = std::max(std::max(prefill_chunk, std::min(max_seqs, kMaxBatch)), 1);
        prefill_o_floats = (prefill_o_floats + 63) & ~size_t(63);
        prefill_ml_floats = (prefill_ml_floats + 63) & ~size_t(63);
        part_o_floats = std::max(part_o_floats, 2 * prefill_o_floats);
        part_ml_floats = std::max(part_ml_floats, 2 * prefill_ml_floats);
        ws.part_o_floats = part_o_floats;
        ws.part_ml_floats = part_ml_floats;
        ws.prefill_o_floats = prefill_o_floats;
        ws.prefill_ml_floats = prefill_ml_floats;
        ws.qprep_slot_elems = size_t(ws.qprep_tokens) * max_q_elems;
        err = cudaMalloc(&ws.qprep, 2 * ws.qprep_slot_elems * 2);
        if (err == cudaSuccess) err = cudaMalloc(&ws.part_o, part_o_floats * sizeof(float));
        if (err == cudaSuccess) err = cudaMalloc(&ws.part_ml, part_ml_floats * sizeof(float));
        // Staging for the host-buffer entry points, two slots: q (twice as wide when the gate is
        // interleaved), gate, out, k, v.
        cache->stage_bytes = (size_t(ws.qprep_tokens) * (4 * max_q_elems + 2 * max_kv_elems) * 4 + 1023) & ~size_t(1023);
        if (err == cudaSuccess) err = cudaMalloc(&cache->stage_dev, 2 * cache->stage_bytes);
        if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&cache->copy_in, cudaStreamNonBlocking);
        if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&cache->copy_out, cudaStreamNonBlocking);
        for (int i = 0; i < 2 && err == cudaSuccess; ++i) {
            err = cudaEventCreateWithFlags(&cache->in_done[i], cudaEventDisableTiming);
            if (err == cudaSuccess) err = cudaEventCreateWithFlags(&cache->step_done[i], cudaEventDisableTiming);
            if (err == cudaSuccess) err = cudaEventCreateWithFlags(&cache->out_done[i], cudaEventDisableTiming);
        }
        if (err == cudaSuccess) err = cudaEventCreateWithFlags(&cache->entry, cudaEventDisableTiming);
        if (err != cudaSuccess) {
            cudaGetLastError();
            st = fail(HC_ALLOC_FAILED, std::string("KV cache workspace: ") + cudaGetErrorString(err));
        }
    }
    if (st != HC_OK) {
        const std::string message = g_last_error;
        hc_kv_cache_destroy(cache);
        g_last_error = message;
        return st;
    }
    *out = cache;
    return HC_OK;
}

void hc_kv_cache_destroy(hc_kv_cache* cache) {
    if (!cache) return;
    for (hc_layer_store& L : cache->layers) {
        if (L.k) cudaFree(L.k);
        if (L.v) cudaFree(L.v);
        tc_free_tensor_maps(L);
    }
    if (cache->ws.qprep) cudaFree(cache->ws.qprep);
    if (cache->ws.part_o) cudaFree(cache->ws.part_o);
    if (cache->ws.part_ml) cudaFree(cache->ws.part_ml);
    if (cache->stage_dev) cudaFree(cache->stage_dev);
    if (cache->pages_dev) cudaFree(cache->pages_dev);
    if (cache->pages_host) cudaFreeHost(cache->pages_host);
    if (cache->copy_in) cudaStreamDestroy(cache->copy_in);
    if (cache->copy_out) cudaStreamDestroy(cache->copy_out);
    for (int i = 0; i < 2; ++i) {
        if (cache->in_done[i]) cudaEventDestroy(cache->in_done[i]);
        if (cache->step_done[i]) cudaEventDestroy(cache->step_done[i]);
        if (cache->out_done[i]) cudaEventDestroy(cache->out_done[i]);
    }
    if (cache->entry) cudaEventDestroy(cache->entry);
    delete cache;
}

size_t hc_kv_cache_bytes(const hc_kv_cache* cache) {
    if (!cache) return 0;
    size_t total = 0;
    for (const hc_layer_store& L : cache->layers) {
        const bool paged = cache->pages_dev != nullptr && L.ring == 0;      // one pool for all sequences
        if (L.keeps_history) total += 2 * size_t(paged ? 1 : cache->max_seqs) * L.desc.kv_heads * L.capacity * L.desc.head_dim * 2;
    }
    return total;
}

int hc_kv_free_pages(const hc_kv_cache* cache) {
    return cache && cache->pages_dev ? int(cache->free_pages.size()) : -1;
}

hc_status hc_kv_layer_info(const hc_kv_cache* cache, int layer, hc_layer_info* out) {
    if (!cache || !out || layer < 0 || layer >= int(cache->layers.size())) return fail(HC_INVALID_ARGUMENT, "bad arguments");
    const hc_layer_store& L = cache->layers[size_t(layer)];
    out->keys = L.k;
    out->values = L.v;
    out->ring_size = L.ring > 0 ? L.desc.window + L.ring_margin : 0;
    out->capacity = L.capacity;
    out->entry_bytes = L.keeps_history ? L.desc.kv_heads * L.desc.head_dim * 2 : 0;
    out->windowed = L.desc.window > 0 ? 1 : 0;
    out->keeps_history = L.keeps_history ? 1 : 0;
    return HC_OK;
}

hc_status hc_kv_read(hc_context* ctx, const hc_kv_cache* cache, int layer, int seq, int position, int tokens,
                     uint16_t* keys_out, uint16_t* values_out) {
    if (!ctx || !cache || layer < 0 || layer >= int(cache->layers.size()) || seq < 0 || seq >= cache->max_seqs ||
        position < 0 || tokens < 0) {
        return fail(HC_INVALID_ARGUMENT, "bad arguments");
    }
    const hc_layer_store& L = cache->layers[size_t(layer)];
    if (!L.keeps_history) return fail(HC_UNSUPPORTED, "a recurrent layer keeps no rows");
    if (L.ring == 0 && position + tokens > cache->context_length) return fail(HC_KV_OVERFLOW, "rows beyond capacity");
    cudaError_t err = cudaDeviceSynchronize();
    if (err != cudaSuccess) return check_cuda(err, "synchronise before reading the cache");
    const CacheView view = view_of(cache, L);
    const int d = L.desc.head_dim, heads = L.desc.kv_heads;
    if (view.map.pages != nullptr) {
        // Paged storage: row by row through the host's copy of the page table.
        const int* table = cache->pages_host + size_t(seq) * cache->pages_per_seq;
        for (int t = 0; t < tokens; ++t) {
            const int pos = position + t;
            const int page = table[pos / kTileKeys];
            for (int h = 0; h < heads; ++h) {
                const size_t dst = (size_t(t) * heads + h) * d;
                if (page < 0) {
                    if (keys_out) std::memset(keys_out + dst, 0, size_t(d) * 2);
                    if (values_out) std::memset(values_out + dst, 0, size_t(d) * 2);
                    continue;
                }
                const size_t src = (size_t(h) * L.capacity + size_t(page) * kTileKeys + pos % kTileKeys) * d;
                if (keys_out) err = cudaMemcpy(keys_out + dst, L.k + src, size_t(d) * 2, cudaMemcpyDeviceToHost);
                if (err == cudaSuccess && values_out) err = cudaMemcpy(values_out + dst, L.v + src, size_t(d) * 2, cudaMemcpyDeviceToHost);
                if (err != cudaSuccess) return check_cuda(err, "reading the cache");
            }
        }
        return HC_OK;
    }
    if (L.ring == 0 && view.map.world <= 1 && tokens > 0) {
        // Linear storage: a head's rows are contiguous; one copy per head, then interleave on the host.
        std::vector<uint16_t> plane(size_t(tokens) * d);
        for (int which = 0; which < 2; ++which) {
            uint16_t* out = which == 0 ? keys_out : values_out;
            if (!out) continue;
            const uint16_t* base = which == 0 ? L.k : L.v;
            for (int h = 0; h < heads; ++h) {
                const size_t src = ((size_t(seq) * heads + h) * L.capacity + position) * d;
                err = cudaMemcpy(plane.data(), base + src, plane.size() * 2, cudaMemcpyDeviceToHost);
                if (err != cudaSuccess) return check_cuda(err, "reading the cache");
                for (int t = 0; t < tokens; ++t) {
                    std::memcpy(out + (size_t(t) * heads + h) * d, plane.data() + size_t(t) * d, size_t(d) * 2);
                }
            }
        }
        return HC_OK;
    }
    for (int t = 0; t < tokens; ++t) {
        const int pos = position + t;
        for (int h = 0; h < heads; ++h) {
            const size_t dst = (size_t(t) * heads + h) * d;
            if (!row_is_local(view.map, pos)) {
                if (keys_out) std::memset(keys_out + dst, 0, size_t(d) * 2);
                if (values_out) std::memset(values_out + dst, 0, size_t(d) * 2);
                continue;
            }
            const size_t src = ((size_t(seq) * heads + h) * L.capacity + row_of_position(view.map, pos)) * d;
            if (keys_out) err = cudaMemcpy(keys_out + dst, L.k + src, size_t(d) * 2, cudaMemcpyDeviceToHost);
            if (err == cudaSuccess && values_out) err = cudaMemcpy(values_out + dst, L.v + src, size_t(d) * 2, cudaMemcpyDeviceToHost);
            if (err != cudaSuccess) return check_cuda(err, "reading the cache");
        }
    }
    return HC_OK;
}

int hc_shard_owner(int world, int position) {
    return world <= 1 ? 0 : (position / kTileKeys) % world;
}

int hc_shard_local_row(int world, int position) {
    RowMap map{0, 0, world, 0, nullptr, 0};
    return row_of_position(map, position);
}

hc_status hc_kv_visible_range(const hc_kv_cache* cache, int layer, int position, int* start, int* count) {
    if (!cache || !start || !count || layer < 0 || layer >= int(cache->layers.size()) || position < 0) {
        return fail(HC_INVALID_ARGUMENT, "bad arguments");
    }
    const hc_layer_store& L = cache->layers[size_t(layer)];
    if (!L.keeps_history) return fail(HC_UNSUPPORTED, "a recurrent layer has no visible range");
    if (L.desc.window == 0) {
        *start = 0;
        *count = position + 1;
        return HC_OK;
    }
    *start = std::max(0, position - L.desc.window + 1);
    *count = position - *start + 1;
    return HC_OK;
}

static bool seq_ok(const hc_kv_cache* cache, int seq) { return cache && seq >= 0 && seq < cache->max_seqs; }

hc_status hc_kv_length(const hc_kv_cache* cache, int seq, int* length) {
    if (!seq_ok(cache, seq) || !length) return fail(HC_INVALID_ARGUMENT, "bad arguments");
    *length = cache->lengths[size_t(seq)];
    return HC_OK;
}

hc_status hc_kv_advance(hc_kv_cache* cache, int seq, int tokens) {
    if (!seq_ok(cache, seq) || tokens < 0) return fail(HC_INVALID_ARGUMENT, "bad arguments");
    const int length = cache->lengths[size_t(seq)] + tokens;
    // Only linear layers can overflow (KVCache.swift:204-212).
    for (const hc_layer_store& L : cache->layers) {
        if (L.keeps_history && L.ring == 0 && length > cache->context_length) {
            return fail(HC_KV_OVERFLOW, "position " + std::to_string(length - 1) + " beyond capacity " +
                                            std::to_string(cache->context_length));
        }
    }
    cache->lengths[size_t(seq)] = length;
    return HC_OK;
}

hc_status hc_kv_reset(hc_kv_cache* cache, int seq) {
    if (!seq_ok(cache, seq)) return fail(HC_INVALID_ARGUMENT, "bad arguments");
    cache->lengths[size_t(seq)] = 0;
    release_pages(cache, seq, 0);
    return HC_OK;
}

hc_status hc_kv_rewind_floor(const hc_kv_cache* cache, int seq, int* floor) {
    if (!seq_ok(cache, seq) || !floor) return fail(HC_INVALID_ARGUMENT, "bad arguments");
    // KVCache.rewindFloor (KVCache.swift:95-99): the smallest ring's margin beyond its window.
    int margin = -1;
    for (const hc_layer_store& L : cache->layers) {
        if (L.keeps_history && L.ring > 0) {
            const int m = L.ring_margin;
            margin = margin < 0 ? m : std::min(margin, m);
        }
    }
    *floor = margin < 0 ? 0 : std::max(0, cache->lengths[size_t(seq)] - margin);
    return HC_OK;
}

int hc_kv_can_rewind(const hc_kv_cache* cache, int seq, int tokens) {
    int floor = 0;
    if (hc_kv_rewind_floor(cache, seq, &floor) != HC_OK) return 0;
    return tokens >= 0 && tokens <= cache->lengths[size_t(seq)] && tokens >= floor;
}

hc_status hc_kv_rewind(hc_kv_cache* cache, int seq, int tokens) {
    if (!seq_ok(cache, seq)) return fail(HC_INVALID_ARGUMENT, "bad arguments");
    if (!hc_kv_can_rewind(cache, seq, tokens)) {
        int floor = 0;
        hc_kv_rewind_floor(cache, seq, &floor);
        return fail(HC_BAD_REWIND, "rewind to " + std::to_string(tokens) + " is outside the history a ring still holds (length " +
                                       std::to_string(cache->lengths[size_t(seq)]) + ", floor " + std::to_string(floor) + ")");
    }
    cache->lengths[size_t(seq)] = tokens;
    release_pages(cache, seq, (tokens + kTileKeys - 1) / kTileKeys);
    return HC_OK;
}

// ---- the kernel protocol --------------------------------------------------------------------------

hc_status hc_kv_append(hc_context* ctx, hc_kv_cache* cache, int layer, int seq, const void* k, const void* v,
                       int tokens, int first_position, const hc_attn_params* params, void* stream) {
    if (!ctx || !k || !v) return fail(HC_INVALID_ARGUMENT, "null context or buffer");
    hc_status st = validate_params(cache, layer, params);
    if (st != HC_OK) return st;
    if (!seq_ok(cache, seq)) return fail(HC_INVALID_ARGUMENT, "sequence index out of range");
    hc_layer_store& L = cache->layers[size_t(layer)];
    st = check_positions(cache, L, first_position, tokens, params);
    if (st != HC_OK) return st;
    st = ensure_pages(cache, L, seq, first_position, tokens, static_cast<cudaStream_t>(stream));
    if (st != HC_OK) return st;
    const size_t row = size_t(params->kv_heads) * params->head_dim;
    for (int start = 0; start < tokens; start += 32768) {
        const int count = std::min(32768, tokens - start);
        PrepArgs args{};
        fill_common(args, params);
        fill_kv_jobs(args, 0, params, offset_rows(k, size_t(start), row, params->io_dtype),
                     offset_rows(v, size_t(start), row, params->io_dtype));
        args.n_jobs = 2;
        args.tokens = count;
        args.first_position = first_position + start;
        args.batched = 0;
        args.seq = seq;
        args.cache = view_of(cache, L);
        st = launch_prepare(ctx, args, static_cast<cudaStream_t>(stream));
        if (st != HC_OK) return st;
    }
    return HC_OK;
}

hc_status hc_kv_append_batch(hc_context* ctx, hc_kv_cache* cache, int layer, const int* seq_ids,
                             const int* positions, int n_seq, const void* k, const void* v,
                             const hc_attn_params* params, void* stream) {
    if (!ctx || !k || !v || !seq_ids || !positions) return fail(HC_INVALID_ARGUMENT, "null context or buffer");
    hc_status st = validate_params(cache, layer, params);
    if (st != HC_OK) return st;
    hc_layer_store& L = cache->layers[size_t(layer)];
    const size_t row = size_t(params->kv_heads) * params->head_dim;
    for (int start = 0; start < n_seq; start += kMaxBatch) {
        const int count = std::min(kMaxBatch, n_seq - start);
        PrepArgs args{};
        fill_common(args, params);
        fill_kv_jobs(args, 0, params, offset_rows(k, size_t(start), row, params->io_dtype),
                     offset_rows(v, size_t(start), row, params->io_dtype));
        args.n_jobs = 2;
        args.tokens = count;
        args.batched = 1;
        for (int b = 0; b < count; ++b) {
            if (!seq_ok(cache, seq_ids[start + b])) return fail(HC_INVALID_ARGUMENT, "sequence index out of range");
            st = check_positions(cache, L, positions[start + b], 1, params);
            if (st == HC_OK) st = ensure_pages(cache, L, seq_ids[start + b], positions[start + b], 1, static_cast<cudaStream_t>(stream));
            if (st != HC_OK) return st;
            args.meta.seq[b] = seq_ids[start + b];
            args.meta.pos[b] = positions[start + b];
        }
        args.cache = view_of(cache, L);
        st = launch_prepare(ctx, args, static_cast<cudaStream_t>(stream));
        if (st != HC_OK) return st;
    }
    return HC_OK;
}

hc_status hc_attention_prefill(hc_context* ctx, hc_kv_cache* cache, int layer, int seq, const void* q, void* out,
                               int tokens, int first_position, const hc_attn_params* params, void* stream) {
    return prefill_impl(ctx, cache, layer, seq, q, out, tokens, first_position, params, false,
                        static_cast<cudaStream_t>(stream));
}

hc_status hc_attention_decode(hc_context* ctx, hc_kv_cache* cache, int layer, const int* seq_ids,
                              const int* positions, int n_seq, const void* q, void* out,
                              const hc_attn_params* params, void* stream) {
    return decode_impl(ctx, cache, layer, seq_ids, positions, n_seq, q, out, params, false,
                       static_cast<cudaStream_t>(stream));
}

size_t hc_attention_partial_bytes(const hc_attn_params* params, int rows) {
    if (!params || rows < 0) return 0;
    return size_t(rows) * params->q_heads * (params->head_dim + 2) * sizeof(float);
}

hc_status hc_attention_prefill_partial(hc_context* ctx, hc_kv_cache* cache, int layer, int seq, const void* q,
                                       void* partial, int tokens, int first_position,
                                       const hc_attn_params* params, void* stream) {
    return prefill_impl(ctx, cache, layer, seq, q, partial, tokens, first_position, params, true,
                        static_cast<cudaStream_t>(stream));
}

hc_status hc_attention_decode_partial(hc_context* ctx, hc_kv_cache* cache, int layer, const int* seq_ids,
                                      const int* positions, int n_seq, const void* q, void* partial,
                                      const hc_attn_params* params, void* stream) {
    return decode_impl(ctx, cache, layer, seq_ids, positions, n_seq, q, partial, params, true,
                       static_cast<cudaStream_t>(stream));
}

hc_status hc_attention_combine(hc_context* ctx, const void* gathered, int world, int rows, const void* q, void* out,
                               const hc_attn_params* params, void* stream) {
    if (!ctx || !gathered || !out || !params) return fail(HC_INVALID_ARGUMENT, "null context or buffer");
    if (world < 1 || rows < 0) return fail(HC_COMM_ERROR, "combine: world must be at least 1");
    EpilogueArgs ep{};
    ep.out = out;
    ep.io_dtype = params->io_dtype;
    ep.write_partial = 0;
    ep.gate_layout = params->gate_layout;
    if (params->gate_layout == HC_GATE_SEPARATE) {
        if (!params->gate) return fail(HC_INVALID_ARGUMENT, "HC_GATE_SEPARATE without a gate buffer");
        ep.gate = params->gate;
    } else if (params->gate_layout == HC_GATE_INTERLEAVED) {
        if (!q) return fail(HC_INVALID_ARGUMENT, "HC_GATE_INTERLEAVED needs q (the gate sits beside the query)");
        ep.gate = q;
    }
    return launch_combine(ctx, static_cast<const float*>(gathered), world, rows, params->q_heads,
                          params->head_dim, ep, static_cast<cudaStream_t>(stream));
}

hc_status hc_rms_norm(hc_context* ctx, const void* x, const void* scale_bf16, void* y, int tokens, int width, float eps,
                      int x_dtype, int y_dtype, void* stream) {
    if (!ctx || !x || !y) return fail(HC_INVALID_ARGUMENT, "null context or buffer");
    if (tokens < 0 || width <= 0) return fail(HC_INVALID_ARGUMENT, "bad sizes");
    if ((x_dtype != HC_F32 && x_dtype != HC_BF16) || (y_dtype != HC_F32 && y_dtype != HC_BF16)) {
        return fail(HC_INVALID_ARGUMENT, "dtypes must be HC_F32 or HC_BF16");
    }
    return launch_rms_norm_rows(ctx, x, static_cast<const uint16_t*>(scale_bf16), y, tokens, width, eps, x_dtype, y_dtype,
                                static_cast<cudaStream_t>(stream));
}

hc_status hc_linear(hc_context* ctx, const void* x, const void* w, const void* bias, const void* residual, void* y,
                    int tokens, int in_features, int out_features, int y_dtype, void* stream) {
    if (!ctx || !x || !w || !y) return fail(HC_INVALID_ARGUMENT, "null context or buffer");
    if (tokens < 0 || in_features <= 0 || out_features <= 0) return fail(HC_INVALID_ARGUMENT, "bad sizes");
    if (y_dtype != HC_F32 && y_dtype != HC_BF16) return fail(HC_INVALID_ARGUMENT, "y_dtype must be HC_F32 or HC_BF16");
    if (in_features % 64 != 0) {
        return fail(HC_DIM_MISMATCH, "hc_linear: in_features " + std::to_string(in_features) + " must be a multiple of 64");
    }
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) & 15) {
        return fail(HC_INVALID_ARGUMENT, "hc_linear: x, w and y must be 16-byte aligned");
    }
    if (residual && y_dtype != HC_F32) return fail(HC_INVALID_ARGUMENT, "hc_linear: a residual needs an fp32 y");
    if (tokens == 0) return HC_OK;
    const float* res = static_cast<const float*>(residual);
    return linear_tc(ctx, x, 1, &w, &bias, &res, &y, &out_features, tokens, in_features, y_dtype,
                     static_cast<cudaStream_t>(stream));
}

hc_status hc_linear_group(hc_context* ctx, const void* x, int n, const void* const* w, const void* const* bias,
                          void* const* y, const int* out_features, int tokens, int in_features, int y_dtype, void* stream) {
    if (!ctx || !x || !w || !y || !out_features) return fail(HC_INVALID_ARGUMENT, "null context or buffer");
    if (n < 1 || n > 4) return fail(HC_INVALID_ARGUMENT, "hc_linear_group takes 1 to 4 projections");
    if (tokens < 0 || in_features <= 0) return fail(HC_INVALID_ARGUMENT, "bad sizes");
    if (y_dtype != HC_F32 && y_dtype != HC_BF16) return fail(HC_INVALID_ARGUMENT, "y_dtype must be HC_F32 or HC_BF16");
    if (in_features % 64 != 0) {
        return fail(HC_DIM_MISMATCH, "hc_linear_group: in_features " + std::to_string(in_features) + " must be a multiple of 64");
    }
    uintptr_t bits = reinterpret_cast<uintptr_t>(x);
    for (int j = 0; j < n; ++j) {
        if (!w[j] || !y[j] || out_features[j] <= 0) return fail(HC_INVALID_ARGUMENT, "hc_linear_group: null weight or output, or a bad width");
        bits |= reinterpret_cast<uintptr_t>(w[j]) | reinterpret_cast<uintptr_t>(y[j]);
    }
    if (bits & 15) return fail(HC_INVALID_ARGUMENT, "hc_linear_group: x, w and y must be 16-byte aligned");
    if (tokens == 0) return HC_OK;
    return linear_tc(ctx, x, n, w, bias, nullptr, y, out_features, tokens, in_features, y_dtype, static_cast<cudaStream_t>(stream));
}

hc_status hc_rms_norm_heads(hc_context* ctx, void* vector, const void* weight_bf16, int tokens, int heads,
                            int head_dim, float eps, int io_dtype, void* stream) {
    if (!ctx || !vector || tokens < 0 || heads <= 0) return fail(HC_INVALID_ARGUMENT, "bad arguments");
    if (head_dim <= 0 || head_dim % 2 != 0 || head_dim > 512) return fail(HC_DIM_MISMATCH, "head_dim must be even and at most 512");
    for (int start = 0; start < tokens; start += 32768) {
        PrepArgs args{};
        args.head_dim = head_dim;
        args.eps = eps;
        PrepJob& job = args.job[0];
        job.src = offset_rows(vector, size_t(start), size_t(heads) * head_dim, io_dtype);
        job.dst = const_cast<void*>(job.src);
        job.src_dtype = io_dtype;
        job.heads = heads;
        job.token_stride = (long long)heads * head_dim;
        job.head_stride = head_dim;
        job.norm = weight_bf16 ? 1 : 2;
        job.weight = static_cast<const uint16_t*>(weight_bf16);
        job.rope = 0;
        job.kind = 3;
        args.n_jobs = 1;
        args.tokens = std::min(32768, tokens - start);
        hc_status st = launch_prepare(ctx, args, static_cast<cudaStream_t>(stream));
        if (st != HC_OK) return st;
    }
    return HC_OK;
}

hc_status hc_apply_rope(hc_context* ctx, void* vector, const hc_rope_table* table, int tokens, int heads,
                        int head_dim, int first_position, int io_dtype, void* stream) {
    if (!ctx || !vector || !table || tokens < 0 || heads <= 0 || first_position < 0) return fail(HC_INVALID_ARGUMENT, "bad arguments");
    if (head_dim <= 0 || head_dim % 2 != 0 || head_dim > 512 || table->pairs != head_dim / 2) {
        return fail(HC_DIM_MISMATCH, "rope table pairs != head_dim / 2");
    }
    if (first_position + tokens > table->positions) return fail(HC_DIM_MISMATCH, "rope table is shorter than the positions asked for");
    for (int start = 0; start < tokens; start += 32768) {
        PrepArgs args{};
        args.head_dim = head_dim;
        args.cos = table->cos;
        args.sin = table->sin;
        args.table_positions = table->positions;
        PrepJob& job = args.job[0];
        job.src = offset_rows(vector, size_t(start), size_t(heads) * head_dim, io_dtype);
        job.dst = const_cast<void*>(job.src);
        job.src_dtype = io_dtype;
        job.heads = heads;
        job.token_stride = (long long)heads * head_dim;
        job.head_stride = head_dim;
        job.norm = 0;
        job.rope = 1;
        job.kind = 3;
        args.n_jobs = 1;
        args.tokens = std::min(32768, tokens - start);
        args.first_position = first_position + start;
        hc_status st = launch_prepare(ctx, args, static_cast<cudaStream_t>(stream));
        if (st != HC_OK) return st;
    }
    return HC_OK;
}

hc_status hc_qwen_split_query_gate(hc_context* ctx, const void* combined, void* query, void* gate, int tokens,
                                   int heads, int head_dim, int io_dtype, void* stream) {
    if (!ctx || !combined || !query || !gate || tokens < 0 || heads <= 0 || head_dim <= 0) return fail(HC_INVALID_ARGUMENT, "bad arguments");
    return launch_split_query_gate(ctx, combined, query, gate, tokens, heads, head_dim, io_dtype,
                                   static_cast<cudaStream_t>(stream));
}

hc_status hc_qwen_apply_output_gate(hc_context* ctx, void* output, const void* gate, size_t count, int io_dtype,
                                    void* stream) {
    if (!ctx || !output || !gate) return fail(HC_INVALID_ARGUMENT, "bad arguments");
    return launch_output_gate(ctx, output, gate, count, io_dtype, static_cast<cudaStream_t>(stream));
}

hc_status hc_layer_step(hc_context* ctx, hc_kv_cache* cache, int layer, int seq, const void* q, const void* k,
                        const void* v, void* out, int tokens, int first_position,
                        const hc_attn_params* params, void* stream) {
    if (!ctx || !q || !k || !v || !out) return fail(HC_INVALID_ARGUMENT, "null context or buffer");
    hc_status st = validate_params(cache, layer, params);
    if (st != HC_OK) return st;
    if (tokens <= 0) return fail(HC_INVALID_ARGUMENT, "tokens must be positive");
    if (tokens > 1 && tokens <= cache->ws.qprep_tokens) {
        // One prologue launch for k, v and q, then the attention kernel.
        return prefill_impl(ctx, cache, layer, seq, q, out, tokens, first_position, params, false,
                            static_cast<cudaStream_t>(stream), k, v);
    }
    if (tokens == 1) {
        if (!seq_ok(cache, seq)) return fail(HC_INVALID_ARGUMENT, "sequence index out of range");
        const int position = first_position;
        return decode_impl(ctx, cache, layer, &seq, &position, 1, q, out, params, false,
                           static_cast<cudaStream_t>(stream), k, v);
    }
    st = hc_kv_append(ctx, cache, layer, seq, k, v, tokens, first_position, params, stream);
    if (st != HC_OK) return st;
    return hc_attention_prefill(ctx, cache, layer, seq, q, out, tokens, first_position, params, stream);
}

hc_status hc_prefill_chunks(hc_context* ctx, hc_kv_cache* cache, int layer, int seq, const void* q, const void* k,
                            const void* v, void* out, int tokens, int first_position, int chunk,
                            const hc_attn_params* params, void* stream) {
    if (!ctx || !q || !k || !v || !out) return fail(HC_INVALID_ARGUMENT, "null context or buffer");
    hc_status st = validate_params(cache, layer, params);
    if (st != HC_OK) return st;
    if (tokens <= 0 || chunk <= 0) return fail(HC_INVALID_ARGUMENT, "tokens and chunk must be positive");
    const int d = params->head_dim;
    const int mult = params->gate_layout == HC_GATE_INTERLEAVED ? 2 : 1;
    // A chunk's prologue (K/V append, query norm and rotation) touches nothing the previous chunk's
    // attention reads, apart from the prepared-query buffer, which has two slots: it runs on a stream
    // of its own, one chunk ahead, in the SMs the attention kernel leaves idle while its last thread
    // blocks finish.  (A ring is stored one margin longer than the reference's, so the rows of chunk
    // i + 1 land on positions older than any key chunk i attends to.)
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const hc_layer_store& L = cache->layers[size_t(layer)];
    const bool ahead_ok = chunk > 1 && chunk <= cache->ws.qprep_tokens && tokens > chunk && cache->copy_in != nullptr &&
                          (L.ring == 0 || L.ring >= L.desc.window + 2 * chunk);
    // Nor does a chunk's attention read anything the previous chunk's attention writes (the workspace
    // for segment partials and second-fold state exists twice): the chunks alternate between the
    // caller's stream and a second one, and a chunk's thread blocks take over the SMs as the previous
    // chunk's thread blocks leave them, instead of waiting for the last one.
    const bool alternate = ahead_ok && cache->copy_out != nullptr;
    if (ahead_ok) {
        cudaError_t err = cudaEventRecord(cache->entry, s);
        if (err == cudaSuccess) err = cudaStreamWaitEvent(cache->copy_in, cache->entry, 0);
        if (err == cudaSuccess && alternate) err = cudaStreamWaitEvent(cache->copy_out, cache->entry, 0);
        if (err != cudaSuccess) return check_cuda(err, "prefill chunks: entry event");
    }
    bool other_used = false;
    int index = 0;
    for (int start = 0; start < tokens; start += chunk, ++index) {
        const int count = std::min(chunk, tokens - start);
        hc_attn_params local = *params;
        if (params->block_ends) local.block_ends = params->block_ends + start;
        if (params->gate_layout == HC_GATE_SEPARATE) {
            local.gate = offset_rows(params->gate, size_t(start), size_t(params->q_heads) * d, params->io_dtype);
        }
        const void* q_rows = offset_rows(q, size_t(start), size_t(params->q_heads) * d * mult, params->io_dtype);
        const void* k_rows = offset_rows(k, size_t(start), size_t(params->kv_heads) * d, params->io_dtype);
        const void* v_rows = offset_rows(v, size_t(start), size_t(params->kv_heads) * d, params->io_dtype);
        void* out_rows = const_cast<unsigned char*>(offset_rows(out, size_t(start), size_t(params->q_heads) * d, params->io_dtype));
        if (ahead_ok && count > 1) {
            const int slot = index & 1;
            // The slot's prepared queries were last read by the attention of chunk index - 2.
            if (index >= 2) {
                const cudaError_t err = cudaStreamWaitEvent(cache->copy_in, cache->step_done[slot], 0);
                if (err != cudaSuccess) return check_cuda(err, "prefill chunks: slot event");
            }
            const PrologueAhead ahead{cache->copy_in, cache->in_done[slot], slot};
            const cudaStream_t attend_on = (alternate && slot == 1) ? cache->copy_out : s;
            other_used = other_used || attend_on != s;
            st = prefill_impl(ctx, cache, layer, seq, q_rows, out_rows, count, first_position + start, &local, false,
                              attend_on, k_rows, v_rows, &ahead);
            if (st != HC_OK) return st;
            const cudaError_t err = cudaEventRecord(cache->step_done[slot], attend_on);
            if (err != cudaSuccess) return check_cuda(err, "prefill chunks: step event");
        } else {
            if (other_used) {
                // A chunk outside the pipeline (a last chunk of one token) follows everything before it.
                const cudaError_t err = cudaStreamWaitEvent(s, cache->step_done[1], 0);
                if (err != cudaSuccess) return check_cuda(err, "prefill chunks: join event");
            }
            st = hc_layer_step(ctx, cache, layer, seq, q_rows, k_rows, v_rows, out_rows, count, first_position + start, &local, stream);
            if (st != HC_OK) return st;
        }
    }
    if (other_used) {
        // The caller's stream ends behind the chunks that ran on the other one.
        const cudaError_t err = cudaStreamWaitEvent(s, cache->step_done[1], 0);
        if (err != cudaSuccess) return check_cuda(err, "prefill chunks: join event");
    }
    return HC_OK;
}

// The body of the host-buffer entry points.  Chunk i's inputs are copied in on one stream while chunk
// i - 1 runs on the caller's stream and chunk i - 2's output is copied back on a third; two staging
// slots, ordered by events.  One cudaMemcpyAsync per buffer.
static hc_status host_chunks(hc_context* ctx, hc_kv_cache* cache, int layer, int seq, const void* q, const void* k,
                             const void* v, void* out, int tokens, int first_position, int chunk,
                             const hc_attn_params* params, cudaStream_t s) {
    const size_t eb = dtype_bytes(params->io_dtype);
    const int d = params->head_dim;
    const int mult = params->gate_layout == HC_GATE_INTERLEAVED ? 2 : 1;
    const bool sep_gate = params->gate_layout == HC_GATE_SEPARATE;
    const size_t q_row = size_t(params->q_heads) * d * mult * eb;
    const size_t kv_row = size_t(params->kv_heads) * d * eb;
    const size_t o_row = size_t(params->q_heads) * d * eb;
    auto align = [](size_t x) { return (x + 255) & ~size_t(255); };
    const size_t off_k = align(q_row * chunk);
    const size_t off_v = off_k + align(kv_row * chunk);
    const size_t off_g = off_v + align(kv_row * chunk);
    const size_t off_o = off_g + (sep_gate ? align(o_row * chunk) : 0);
    if (off_o + o_row * chunk > cache->stage_bytes) return fail(HC_KV_OVERFLOW, "staging buffer too small for this chunk");
    // The copies may start once the work already in the caller's stream has been reached.
    cudaError_t err = cudaEventRecord(cache->entry, s);
    if (err == cudaSuccess) err = cudaStreamWaitEvent(cache->copy_in, cache->entry, 0);
    if (err != cudaSuccess) return check_cuda(err, "host step: entry event");
    const unsigned char* hq = static_cast<const unsigned char*>(q);
    const unsigned char* hk = static_cast<const unsigned char*>(k);
    const unsigned char* hv = static_cast<const unsigned char*>(v);
    const unsigned char* hg = static_cast<const unsigned char*>(params->gate);
    unsigned char* ho = static_cast<unsigned char*>(out);
    int index = 0;
    for (int start = 0; start < tokens; start += chunk, ++index) {
        const int count = std::min(chunk, tokens - start);
        const int slot = index & 1;
        unsigned char* base = static_cast<unsigned char*>(cache->stage_dev) + size_t(slot) * cache->stage_bytes;
        // The slot's previous occupant (chunk index - 2) must have run and its output left.
        if (index >= 2) {
            err = cudaStreamWaitEvent(cache->copy_in, cache->out_done[slot], 0);
            if (err != cudaSuccess) return check_cuda(err, "host step: slot reuse");
        }
        err = cudaMemcpyAsync(base, hq + size_t(start) * q_row, q_row * count, cudaMemcpyHostToDevice, cache->copy_in);
        if (err == cudaSuccess) err = cudaMemcpyAsync(base + off_k, hk + size_t(start) * kv_row, kv_row * count, cudaMemcpyHostToDevice, cache->copy_in);
        if (err == cudaSuccess) err = cudaMemcpyAsync(base + off_v, hv + size_t(start) * kv_row, kv_row * count, cudaMemcpyHostToDevice, cache->copy_in);
        if (err == cudaSuccess && sep_gate) err = cudaMemcpyAsync(base + off_g, hg + size_t(start) * o_row, o_row * count, cudaMemcpyHostToDevice, cache->copy_in);
        if (err == cudaSuccess) err = cudaEventRecord(cache->in_done[slot], cache->copy_in);
        if (err == cudaSuccess) err = cudaStreamWaitEvent(s, cache->in_done[slot], 0);
        if (err != cudaSuccess) return check_cuda(err, "host to device copy");
        hc_attn_params local = *params;
        if (params->block_ends) local.block_ends = params->block_ends + start;    // device memory, like the sinks
        if (sep_gate) local.gate = base + off_g;
        const hc_status st = hc_layer_step(ctx, cache, layer, seq, base, base + off_k, base + off_v, base + off_o, count,
                                           first_position + start, &local, s);
        if (st != HC_OK) return st;
        err = cudaEventRecord(cache->step_done[slot], s);
        if (err == cudaSuccess) err = cudaStreamWaitEvent(cache->copy_out, cache->step_done[slot], 0);
        if (err == cudaSuccess) err = cudaMemcpyAsync(ho + size_t(start) * o_row, base + off_o, o_row * count, cudaMemcpyDeviceToHost, cache->copy_out);
        if (err == cudaSuccess) err = cudaEventRecord(cache->out_done[slot], cache->copy_out);
        if (err != cudaSuccess) return check_cuda(err, "device to host copy");
    }
    // The call returns when the results are on the host.
    err = cudaStreamSynchronize(cache->copy_out);
    if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    if (err != cudaSuccess) return check_cuda(err, "host step: synchronise");
    return HC_OK;
}

hc_status hc_layer_step_host(hc_context* ctx, hc_kv_cache* cache, int layer, int seq, const void* q, const void* k,
                             const void* v, void* out, int tokens, int first_position,
                             const hc_attn_params* params, void* stream) {
    if (!ctx || !q || !k || !v || !out) return fail(HC_INVALID_ARGUMENT, "null context or buffer");
    hc_status st = validate_params(cache, layer, params);
    if (st != HC_OK) return st;
    if (tokens <= 0) return fail(HC_INVALID_ARGUMENT, "tokens must be positive");
    if (tokens > cache->ws.qprep_tokens) {
        return fail(HC_KV_OVERFLOW, "hc_layer_step_host takes at most " + std::to_string(cache->ws.qprep_tokens) + " tokens per call");
    }
    return host_chunks(ctx, cache, layer, seq, q, k, v, out, tokens, first_position, tokens, params,
                       static_cast<cudaStream_t>(stream));
}

hc_status hc_prefill_host(hc_context* ctx, hc_kv_cache* cache, int layer, int seq, const void* q, const void* k,
                          const void* v, void* out, int tokens, int first_position, int chunk,
                          const hc_attn_params* params, void* stream) {
    if (!ctx || !q || !k || !v || !out) return fail(HC_INVALID_ARGUMENT, "null context or buffer");
    hc_status st = validate_params(cache, layer, params);
    if (st != HC_OK) return st;
    if (tokens <= 0 || chunk <= 0) return fail(HC_INVALID_ARGUMENT, "tokens and chunk must be positive");
    if (chunk > cache->ws.qprep_tokens) {
        return fail(HC_KV_OVERFLOW, "hc_prefill_host takes chunks of at most " + std::to_string(cache->ws.qprep_tokens) + " tokens");
    }
    return host_chunks(ctx, cache, layer, seq, q, k, v, out, tokens, first_position, chunk, params,
                       static_cast<cudaStream_t>(stream));
}

}  // extern "C"
