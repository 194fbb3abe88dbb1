// internal.hpp — host-side objects behind the opaque handles of hydra_cuda.h, and the launchers
// each .cu file exports to api.cu.  Nothing here is visible outside the shared library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/hydra_cuda.h"
#include "common.cuh"

namespace hc {

// At most this many sequences share one decode launch; larger batches are cut into launches.
constexpr int kMaxBatch = 64;

struct BatchMeta {
    int seq[kMaxBatch];
    int pos[kMaxBatch];
};

// One head's rows of one layer, as the kernels address them.
struct CacheView {
    uint16_t* k;       // bf16 [max_seqs][kv_heads][capacity][head_dim]
    uint16_t* v;
    int capacity;      // rows per (sequence, head)
    int kv_heads;
    RowMap map;
};

struct AttnShape {
    int q_heads;
    int kv_heads;
    int head_dim;
    int group;          // q_heads / kv_heads
    int window;         // 0 = full
    float c;            // sm_scale * log2(e)
    const uint16_t* sinks;  // bf16 [q_heads] or null
    int count_sink;     // 0 on ranks > 0 of a sequence-sharded cache
};

// What the prologue does to one of q, k, v.
// Launch with programmatic stream serialisation allowed (see pdl_wait in common.cuh).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

struct PrepJob {
    const void* src;
    int src_dtype;
    int heads;
    long long token_stride;  // elements between tokens in src
    int head_stride;         // elements between heads in src (2 * d for an interleaved gate)
    int norm;                // 0 none, 1 weighted, 2 weightless
    const uint16_t* weight;
    int rope;                // 0 / 1
    int kind;                // 0: dense bf16 [tokens][heads][d]; 1: K rows; 2: V rows; 3: in place
    void* dst;
};
struct PrepArgs {
    PrepJob job[3];
    int n_jobs;
    int head_dim;
    float eps;
    const float* cos;        // fp32 [table_positions][head_dim / 2]
    const float* sin;
    int table_positions;
    int tokens;
    int first_position;      // position of token 0 when batched == 0
    int batched;             // 1: token t is sequence meta.seq[t] at position meta.pos[t]
    int seq;                 // sequence when batched == 0
    CacheView cache;         // for kinds 1 and 2
    BatchMeta meta;
};

struct EpilogueArgs {
    void* out;               // [rows][q_heads][d] io dtype, or fp32 partial [rows][q_heads][d + 2]
    int io_dtype;
    int write_partial;       // 1: write (A, M, L) instead of the finished value
    int gate_layout;
    const void* gate;        // HC_GATE_SEPARATE: [rows][q_heads][d]; INTERLEAVED: q_proj output
};

struct Workspace {
    uint16_t* qprep = nullptr;   // bf16 [2][qprep_tokens][q_heads][d]: two slots, so that a chunk's prologue can
                                 // run while the previous chunk's attention still reads its queries
    size_t qprep_slot_elems = 0; // elements of one slot
    int qprep_tokens = 0;
    float* part_o = nullptr;     // fp32 [rows][slots][d]: segment partials, rows and slots those of the call
    float* part_ml = nullptr;    // fp32 [rows][slots][2]
    size_t part_o_floats = 0;    // capacities
    size_t part_ml_floats = 0;
    // What a prefill launch can need of the two (segment partials or second-fold state): the buffers
    // hold it twice, so that two chunks' attention launches may be in flight at once, the second one
    // working in the upper halves [prefill_o_floats, 2 prefill_o_floats) and likewise for part_ml.
    size_t prefill_o_floats = 0;
    size_t prefill_ml_floats = 0;
};

}  // namespace hc

struct hc_context {
    int device = 0;
    int sm_count = 0;
    uint64_t launches = 0;
    int* status_dev = nullptr;    // one word the kernels may set on a bounded-wait timeout
    int* status_host = nullptr;   // pinned mirror
    float* static_scratch = nullptr;   // device address of the fixed scratch of hc_attention_decode_static
};

struct hc_rope_table {
    int device = 0;
    float* cos = nullptr;
    float* sin = nullptr;
    int positions = 0;
    int pairs = 0;
};

struct hc_layer_store {
    hc_layer_desc desc{};
    uint16_t* k = nullptr;
    uint16_t* v = nullptr;
    int ring = 0;                 // rows of the ring as stored (0: linear); positions map to pos % ring
    int ring_margin = 0;          // the reference's ring is window + ring_margin rows: what a chunk may
                                  // append at once and how far a rewind may reach
    int capacity = 0;
    int log_segment = 0;          // key tiles per segment, as a power of two (see common.cuh)
    bool keeps_history = false;
    void* tmap_k = nullptr;       // tensor maps of the tcgen05 path (host copies), or null
    void* tmap_v = nullptr;
};

struct hc_kv_cache {
    hc_context* ctx = nullptr;
    std::vector<hc_layer_store> layers;
    int context_length = 0;
    int prefill_chunk = 0;
    int max_seqs = 0;
    hc_shard_desc shard{HC_SHARD_NONE, 0, 1};
    std::vector<int> lengths;
    // Paged storage (hc_kv_cache_create_paged): the linear layers are pools of total_pages pages of 128
    // rows shared by all sequences; one page table for all layers, [max_seqs][pages_per_seq], -1 =
    // not assigned (the device copy holds 0 there: a valid page that no visible key maps to).
    int total_pages = 0;
    int pages_per_seq = 0;
    int* pages_dev = nullptr;
    int* pages_host = nullptr;    // pinned mirror, the source of the asynchronous updates
    std::vector<int> free_pages;
    hc::Workspace ws;
    // hc_layer_step_host / hc_prefill_host: two device staging slots, a stream for the copies in and
    // one for the copies out, and the events that order them against the caller's stream.
    void* stage_dev = nullptr;
    size_t stage_bytes = 0;       // of one slot
    cudaStream_t copy_in = nullptr;
    cudaStream_t copy_out = nullptr;
    cudaEvent_t in_done[2] = {nullptr, nullptr};
    cudaEvent_t step_done[2] = {nullptr, nullptr};
    cudaEvent_t out_done[2] = {nullptr, nullptr};
    cudaEvent_t entry = nullptr;
};

namespace hc {

// Sets the thread's error message and returns `status`.
hc_status fail(hc_status status, const std::string& message);
hc_status check_cuda(cudaError_t err, const char* what);

// prologue.cu
hc_status launch_prepare(hc_context* ctx, const PrepArgs& args, cudaStream_t stream);
hc_status launch_rms_norm_rows(hc_context* ctx, const void* x, const uint16_t* scale, void* out, int tokens, int width,
                               float eps, int x_dtype, int out_dtype, cudaStream_t stream);
hc_status launch_split_query_gate(hc_context* ctx, const void* combined, void* query, void* gate,
                                  int tokens, int heads, int d, int dtype, cudaStream_t stream);
hc_status launch_output_gate(hc_context* ctx, void* output, const void* gate, size_t count,
                             int dtype, cudaStream_t stream);

// attn_simt.cu
hc_status simt_prefill(hc_context* ctx, const AttnShape& shape, const CacheView& cache, int seq,
                       const uint16_t* q, int tokens, int first_position, const EpilogueArgs& ep,
                       cudaStream_t stream, const int* block_ends = nullptr);
hc_status simt_decode(hc_context* ctx, const AttnShape& shape, const CacheView& cache,
                      const BatchMeta& meta, int n_seq, const uint16_t* q, const Workspace& ws,
                      const EpilogueArgs& ep, cudaStream_t stream);
// How a decode launch cuts its rows' keys (see TcArgs in tc_common.cuh for the three ways).
struct DecodePlan {
    int finish;          // whole rows per item, finished by the kernel itself
    int log_run;         // tile partials: items are aligned runs of 2^log_run tiles
    int run_segments;    // segment partials: about this many segments per item
    int tile_partials;   // the kernel writes one partial per tile (log_run < log_segment) rather than per segment
    int slots;           // partial slots per row
    int tiles;           // key tiles of the longest row (on this rank)
};
// The coarsest cut that gives at least target_items items, runs of max_run_segments segments at most.
DecodePlan plan_decode(const AttnShape& shape, const RowMap& map, const BatchMeta& meta, int n_seq, int target_items,
                       bool allow_whole, int max_run_segments);
// The cuts simt_decode and tc_decode make (the latter given the room for partials or row state).
DecodePlan simt_plan_decode(const hc_context* ctx, const AttnShape& shape, const RowMap& map, const BatchMeta& meta, int n_seq);
DecodePlan tc_plan_decode(const hc_context* ctx, const AttnShape& shape, const RowMap& map, const BatchMeta& meta, int n_seq,
                          size_t part_o_floats);
// Both folds (tile partials) or the second fold (segment partials) over the partials in `ws`, then the
// epilogue: for the rows of a decode batch, or for the query tokens of a prefill chunk.
hc_status launch_merge_decode(hc_context* ctx, const AttnShape& shape, const RowMap& map, const BatchMeta& meta,
                              int n_seq, const Workspace& ws, const DecodePlan& plan, const EpilogueArgs& ep,
                              cudaStream_t stream);
hc_status launch_merge_prefill(hc_context* ctx, const AttnShape& shape, const RowMap& map, int tokens,
                               int first_position, const Workspace& ws, int slots, const EpilogueArgs& ep,
                               cudaStream_t stream);
hc_status launch_combine(hc_context* ctx, const float* gathered, int world, int rows, int q_heads,
                         int d, const EpilogueArgs& ep, cudaStream_t stream);
// Device address of the fixed scratch array on `device` (which must be current).
hc_status static_scratch_prepare(int device, float** address);

// attn_tc.cu
// A tensor map (CUtensorMap behind `map`) over a row-major bf16 matrix: boxes of 64 columns x box_rows
// rows, 128-byte swizzle, zeros beyond the edges.
hc_status tc_encode_2d(void* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);
bool tc_supported(const AttnShape& shape);
hc_status tc_prefill(hc_context* ctx, const AttnShape& shape, const hc_layer_store& layer,
                     const CacheView& cache, int seq, const uint16_t* q, int tokens,
                     int first_position, const Workspace& ws, const EpilogueArgs& ep, cudaStream_t stream, const int* block_ends = nullptr);
hc_status tc_decode(hc_context* ctx, const AttnShape& shape, const hc_layer_store& layer,
                    const CacheView& cache, const BatchMeta& meta, int n_seq, const uint16_t* q,
                    const Workspace& ws, const EpilogueArgs& ep, cudaStream_t stream);
// linear_tc.cu
// n_jobs (1 to 4) projections of the same x in one launch; bias / residual may be null, or hold nulls.
hc_status linear_tc(hc_context* ctx, const void* x, int n_jobs, const void* const* w, const void* const* bias,
                    const float* const* residual, void* const* y, const int* out_features, int tokens, int in_features,
                    int y_dtype, cudaStream_t stream);
// attn_tc256.cu (args_ptr: the TcArgs of tc_common.cuh)
hc_status launch_tc256(hc_context* ctx, const void* tmap_k, const void* tmap_v, const void* args_ptr,
                       int n_items, cudaStream_t stream);
hc_status tc_make_tensor_maps(hc_kv_cache* cache, hc_layer_store& layer);
void tc_free_tensor_maps(hc_layer_store& layer);

}  // namespace hc
