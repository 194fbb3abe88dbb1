// shard.cu — the multi-GPU entry points: a shard object that holds this rank's place in an NCCL
// communicator, and sequence-sharded attention as ONE call (partial -> all-gather -> combine, all
// enqueued on the caller's stream).  The reference runs on one device and has no counterpart; the
// merge the combine performs is the log-sum-exp merge of its split decode
// (Sources/HydraMetal/Shaders/attention.metal:418-452), over ranks instead of key chunks.
//
// The exchange is NCCL's all-gather into this GPU's own memory; no kernel here reads a peer's
// memory.  The partials are small (head_dim + 2 floats per query row and head, 16.5 KB per rank for
// a Qwen-shaped decode step), so the collective is latency-bound and one call per step is the
// whole cost.
//
// hc_linear_sharded is the other exchange of a sharded layer: the row-parallel output projection,
// a GEMM per rank and NCCL's sum of the partial results (ReferenceLayer.decode's `hidden +=
// attention W_o^T + b_o`, Sources/HydraReference/ReferenceLayer.swift:186-187, over ranks).

#include <new>

#include "internal.hpp"

#ifdef HC_HAVE_NCCL
#include <nccl.h>
#endif

struct hc_shard {
    hc_context* ctx = nullptr;
    hc_shard_desc desc{HC_SHARD_NONE, 0, 1};
    void* comm = nullptr;            // ncclComm_t, owned by the caller
    float* mine = nullptr;           // this rank's partial
    float* gathered = nullptr;       // [world] partials
    size_t partial_bytes = 0;        // capacity of `mine`
};

using namespace hc;

namespace {

#ifdef HC_HAVE_NCCL
hc_status check_nccl(ncclResult_t result, const char* what) {
    if (result == ncclSuccess) return HC_OK;
    return fail(HC_COMM_ERROR, std::string(what) + ": " + ncclGetErrorString(result));
}
#endif

// Steps 2 and 3 of a sequence-sharded call: gather the ranks' partials, then the combine every rank runs.
hc_status gather_and_combine(hc_context* ctx, hc_shard* shard, int rows, const void* q, void* out,
                             const hc_attn_params* params, void* stream) {
#ifdef HC_HAVE_NCCL
    const size_t count = hc_attention_partial_bytes(params, rows) / sizeof(float);
    hc_status st = check_nccl(ncclAllGather(shard->mine, shard->gathered, count, ncclFloat,
                                            static_cast<ncclComm_t>(shard->comm), static_cast<cudaStream_t>(stream)),
                              "ncclAllGather of the attention partials");
    if (st != HC_OK) return st;
    return hc_attention_combine(ctx, shard->gathered, shard->desc.world, rows, q, out, params, stream);
#else
    (void)ctx; (void)shard; (void)rows; (void)q; (void)out; (void)params; (void)stream;
    return fail(HC_UNSUPPORTED, "this build of the library has no NCCL");
#endif
}

hc_status check_call(hc_context* ctx, hc_shard* shard, hc_kv_cache* cache, const hc_attn_params* params, int rows) {
    if (!ctx || !shard || !cache || !params) return fail(HC_INVALID_ARGUMENT, "null context, shard, cache or params");
    if (cache->shard.mode != shard->desc.mode || cache->shard.rank != shard->desc.rank ||
        cache->shard.world != shard->desc.world) {
        return fail(HC_COMM_ERROR, "the cache was not created with this shard's description (hc_shard_describe)");
    }
    if (hc_attention_partial_bytes(params, rows) > shard->partial_bytes) {
        return fail(HC_KV_OVERFLOW, "this call's partial (" + std::to_string(hc_attention_partial_bytes(params, rows)) +
                                        " B) exceeds what the shard was created for (" +
                                        std::to_string(shard->partial_bytes) + " B)");
    }
    return HC_OK;
}

}  // namespace

extern "C" {

hc_status hc_shard_create(hc_context* ctx, void* nccl_comm, int mode, int rank, int world, size_t max_partial_bytes,
                          hc_shard** out) {
    // The description is checked before anything touches a device, so that a host can validate its
    // rank bookkeeping without one.
    if (world < 1 || rank < 0 || rank >= world || mode < HC_SHARD_NONE || mode > HC_SHARD_SEQUENCE) {
        return fail(HC_COMM_ERROR, "inconsistent shard description: mode " + std::to_string(mode) + ", rank " +
                                       std::to_string(rank) + " of " + std::to_string(world));
    }
    if (!ctx || !out) return fail(HC_INVALID_ARGUMENT, "null context or out pointer");
    *out = nullptr;
    const bool exchanges = mode == HC_SHARD_SEQUENCE && world > 1;
    if (exchanges && !nccl_comm) return fail(HC_COMM_ERROR, "a sequence shard over several ranks needs an NCCL communicator");
#ifdef HC_HAVE_NCCL
    if (nccl_comm && world > 1) {          // a head shard may bring one too, for hc_linear_sharded
        int count = 0, user_rank = -1;
        hc_status st = check_nccl(ncclCommCount(static_cast<ncclComm_t>(nccl_comm), &count), "ncclCommCount");
        if (st == HC_OK) st = check_nccl(ncclCommUserRank(static_cast<ncclComm_t>(nccl_comm), &user_rank), "ncclCommUserRank");
        if (st != HC_OK) return st;
        if (count != world || user_rank != rank) {
            return fail(HC_COMM_ERROR, "the communicator says rank " + std::to_string(user_rank) + " of " + std::to_string(count) +
                                           ", the caller rank " + std::to_string(rank) + " of " + std::to_string(world));
        }
    }
#else
    if (exchanges) return fail(HC_UNSUPPORTED, "this build of the library has no NCCL");
#endif
    hc_shard* shard = new (std::nothrow) hc_shard();
    if (!shard) return fail(HC_ALLOC_FAILED, "out of host memory");
    shard->ctx = ctx;
    shard->desc = hc_shard_desc{world == 1 ? HC_SHARD_NONE : mode, rank, world};
    shard->comm = nccl_comm;
    shard->partial_bytes = exchanges ? max_partial_bytes : 0;
    if (exchanges && max_partial_bytes > 0) {
        cudaError_t err = cudaSetDevice(ctx->device);
        if (err == cudaSuccess) err = cudaMalloc(&shard->mine, max_partial_bytes);
        if (err == cudaSuccess) err = cudaMalloc(&shard->gathered, size_t(world) * max_partial_bytes);
        if (err != cudaSuccess) {
            cudaGetLastError();
            hc_shard_destroy(shard);
            return fail(HC_ALLOC_FAILED, std::string("shard exchange buffers: ") + cudaGetErrorString(err));
        }
    }
    *out = shard;
    return HC_OK;
}

void hc_shard_destroy(hc_shard* shard) {
    if (!shard) return;
    if (shard->mine) cudaFree(shard->mine);
    if (shard->gathered) cudaFree(shard->gathered);
    delete shard;
}

hc_status hc_shard_describe(const hc_shard* shard, hc_shard_desc* desc) {
    if (!shard || !desc) return fail(HC_INVALID_ARGUMENT, "null shard or description");
    *desc = shard->desc;
    return HC_OK;
}

hc_status hc_attention_decode_sharded(hc_context* ctx, hc_shard* shard, hc_kv_cache* cache, int layer,
                                      const int* seq_ids, const int* positions, int n_seq, const void* q, void* out,
                                      const hc_attn_params* params, void* stream) {
    if (shard && shard->desc.mode != HC_SHARD_SEQUENCE) {
        // Head shards (and a world of one) exchange nothing inside attention.
        return hc_attention_decode(ctx, cache, layer, seq_ids, positions, n_seq, q, out, params, stream);
    }
    hc_status st = check_call(ctx, shard, cache, params, n_seq);
    if (st != HC_OK) return st;
    st = hc_attention_decode_partial(ctx, cache, layer, seq_ids, positions, n_seq, q, shard->mine, params, stream);
    if (st != HC_OK) return st;
    return gather_and_combine(ctx, shard, n_seq, q, out, params, stream);
}

hc_status hc_attention_prefill_sharded(hc_context* ctx, hc_shard* shard, hc_kv_cache* cache, int layer, int seq,
                                       const void* q, void* out, int tokens, int first_position,
                                       const hc_attn_params* params, void* stream) {
    if (shard && shard->desc.mode != HC_SHARD_SEQUENCE) {
        return hc_attention_prefill(ctx, cache, layer, seq, q, out, tokens, first_position, params, stream);
    }
    hc_status st = check_call(ctx, shard, cache, params, tokens);
    if (st != HC_OK) return st;
    st = hc_attention_prefill_partial(ctx, cache, layer, seq, q, shard->mine, tokens, first_position, params, stream);
    if (st != HC_OK) return st;
    return gather_and_combine(ctx, shard, tokens, q, out, params, stream);
}

// The output projection of a head-sharded layer: every rank holds the attention output of its own
// heads, [tokens][in_features] with in_features = its heads x head_dim, and the matching columns of
// W_o as a matrix of its own, [out_features][in_features].  Each rank's GEMM gives a partial sum of
// every output element; rank 0's carries the bias and the residual; NCCL adds the partials on the
// caller's stream.
hc_status hc_linear_sharded(hc_context* ctx, hc_shard* shard, const void* x, const void* w, const void* bias,
                            const void* residual, void* y, int tokens, int in_features, int out_features, int scatter,
                            void* stream) {
    if (!shard) return fail(HC_INVALID_ARGUMENT, "null shard");
    const int world = shard->desc.world;
    if (world <= 1) return hc_linear(ctx, x, w, bias, residual, y, tokens, in_features, out_features, HC_F32, stream);
    if (!shard->comm) return fail(HC_COMM_ERROR, "hc_linear_sharded: the shard was created without an NCCL communicator");
    if (scatter && tokens % world != 0) {
        return fail(HC_DIM_MISMATCH, "hc_linear_sharded: " + std::to_string(tokens) + " tokens do not divide over " +
                                         std::to_string(world) + " ranks");
    }
    const bool first = shard->desc.rank == 0;
    hc_status st = hc_linear(ctx, x, w, first ? bias : nullptr, first ? residual : nullptr, y, tokens, in_features,
                             out_features, HC_F32, stream);
    if (st != HC_OK || tokens == 0) return st;
#ifdef HC_HAVE_NCCL
    float* sums = static_cast<float*>(y);
    const size_t count = size_t(tokens) * size_t(out_features);
    if (scatter) {
        const size_t mine = count / size_t(world);
        return check_nccl(ncclReduceScatter(sums, sums + size_t(shard->desc.rank) * mine, mine, ncclFloat, ncclSum,
                                            static_cast<ncclComm_t>(shard->comm), static_cast<cudaStream_t>(stream)),
                          "ncclReduceScatter of the output projection");
    }
    return check_nccl(ncclAllReduce(sums, sums, count, ncclFloat, ncclSum, static_cast<ncclComm_t>(shard->comm),
                                    static_cast<cudaStream_t>(stream)),
                      "ncclAllReduce of the output projection");
#else
    return fail(HC_UNSUPPORTED, "this build of the library has no NCCL");
#endif
}

}  // extern "C"
