// common.cuh — arithmetic shared by every attention kernel in this library.
//
// The kernels agree bit for bit with one another only because they all go through the functions in
// this header: the same exp2, the same rounding of the softmax weights to bf16, the same fold.
// Every floating-point step uses an explicit round-to-nearest intrinsic so that the compiler cannot
// contract or reassociate it differently in two kernels.
//
// The canonical computation (what "attention of one query row" means here):
//
//   keys are cut into tiles of 128 absolute positions: tile j = [128 j, 128 j + 128);
//   for each tile that holds a visible key, the tile partial is
//       s_k  = q . K_k                       (fp32 accumulate over bf16 inputs)
//       m    = max over visible k of s_k
//       p_k  = bf16( exp2( fma(s_k, c, -(m * c)) ) ) for visible k, 0 otherwise;  c = sm_scale * log2(e)
//       l    = sum_k p_k ,  O = sum_k p_k V_k                              (fp32)
//       mm   = m * c
//   tiles are grouped into segments of 2^log_segment consecutive tiles, absolute like the tiles
//   (1024 or 4096 keys; a property of the layer, fixed when its cache is created).  A segment's
//   partial is a left fold over its tiles that hold a visible key, in ascending order, from the
//   empty state:
//       (M, L, A) = (-1e30, 0, 0)
//       Mn = max(M, mm); a = exp2(M - Mn); b = exp2(mm - Mn)
//       L = fma(L, a, l * b);  A = fma(A, a, O * b);  M = Mn
//   and the row's result is the same fold over its segments' partials (M, L, A) in ascending
//   order, seeded with the sink:
//       (M, L, A) = (sink * log2(e), 1, 0)             -- "no sink" is sink = bf16(-1e30)
//       out = A / L, then * sigmoid(gate) when gated.
//   Folding an empty partial changes nothing, exactly, so it does not matter whether a kernel
//   visits a segment in which a row sees no key.
//
// Seeding with the sink is the reference's own construction
// (Sources/HydraMetal/Shaders/attention.metal:156-165): the sink adds to the denominator only.
// A tile partial does not depend on which kernel, which chunk or which split produced it, and the
// two folds visit tiles and segments in the same order everywhere.  So the work of a row may be cut
// anywhere without changing a bit of the result: a thread block may take the whole row and run both
// folds, or one segment and leave the second fold to a merge kernel, or a few tiles and leave both
// folds to it; chunked prefill, token-by-token decode and every such split agree as long as they
// share the tile-partial routine.  Small segments are what lets a prefill launch with few rows
// spread one row's keys over several thread blocks at little cost in partials; large segments keep
// the second fold rare where whole rows already fill the machine.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hc {

constexpr int kTileKeys = 128;
constexpr float kLog2e = 1.4426950408889634f;
// The reference's "unreachable sink": bf16(-1e30) (Sources/HydraMetal/Gemma4LayerRunner.swift:43-49).
constexpr uint16_t kNoSinkBits = 0xF14A;  // bf16 nearest to -1e30 (-1.00026e30)
// Seed of a fold that must not count the sink (ranks > 0 of a sequence-sharded cache).
constexpr float kEmptyMax = -1.0e30f;

// Programmatic dependent launch.  The hot kernels are launched with the stream-serialisation
// attribute relaxed, so a kernel's blocks may be scheduled (and run their set-up) while the kernel
// before it in the stream is still finishing.  Each of them lets its successor go at its very top
// and waits for its predecessors (all of them: the wait is for full completion, memory included)
// before it touches global memory.  Launched the ordinary way the two instructions do nothing.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t bits) {
    return __uint_as_float(uint32_t(bits) << 16);
}
__device__ __forceinline__ uint16_t float_to_bf16_bits(float value) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(value));
}
__device__ __forceinline__ float round_to_bf16(float value) {
    return bf16_bits_to_float(float_to_bf16_bits(value));
}

// Softmax weight of one logit inside its tile, before rounding: exp2( s * c - m * c ), one fused
// multiply-add with neg_mc = -(m * c).  A masked logit (-inf) gives exactly 0.
__device__ __forceinline__ float tile_weight_raw(float s, float neg_mc, float c) {
    return ex2(__fmaf_rn(s, c, neg_mc));
}
__device__ __forceinline__ float tile_weight(float s, float neg_mc, float c) {
    return round_to_bf16(tile_weight_raw(s, neg_mc, c));
}

// One step of the fold: the coefficients, then the update of any accumulated quantity.
__device__ __forceinline__ void fold_coefficients(float M, float mm, float& Mn, float& a, float& b) {
    Mn = fmaxf(M, mm);
    a = ex2(__fsub_rn(M, Mn));
    b = ex2(__fsub_rn(mm, Mn));
}
__device__ __forceinline__ float fold_value(float acc, float a, float part, float b) {
    return __fmaf_rn(acc, a, __fmul_rn(part, b));
}

__device__ __forceinline__ float sigmoid_gate(float g) {
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, ex2(__fmul_rn(-g, kLog2e))));
}
// The last step of a row: the correctly rounded reciprocal of the denominator (one per row; the
// compiler shares it between the row's elements) times the numerator, then the optional gate.
__device__ __forceinline__ float finish_value(float A, float L, bool gated, float g) {
    float out = __fmul_rn(A, __frcp_rn(L));
    if (gated) out = __fmul_rn(out, sigmoid_gate(g));
    return out;
}

// Activations are fp32 or bf16; these two read and write one element of either.
__device__ __forceinline__ float load_io(const void* base, size_t index, int dtype) {
    return dtype == 0 ? reinterpret_cast<const float*>(base)[index]
                      : bf16_bits_to_float(reinterpret_cast<const uint16_t*>(base)[index]);
}
__device__ __forceinline__ void store_io(void* base, size_t index, int dtype, float value) {
    if (dtype == 0) reinterpret_cast<float*>(base)[index] = value;
    else reinterpret_cast<uint16_t*>(base)[index] = float_to_bf16_bits(value);
}

// Where position `pos` of a sequence lives inside one head's rows of the cache, and how the layer
// groups its key tiles into segments.
//   ring > 0            : physical = pos % ring                      (ring is a multiple of 128)
//   world > 1 (sequence): tile j = pos / 128 belongs to rank j % world and is that rank's local
//                         tile j / world
//   log_segment         : a segment is 2^log_segment consecutive tiles, absolute like the tiles
//                         (3 or 5: 1024 or 4096 keys; fixed per layer when the cache is created)
//   pages != null       : paged storage: the cache is a pool of 128-row pages shared by all sequences,
//                         and key tile j of sequence s lives in page pages[s * pages_per_seq + j]
struct RowMap {
    int ring;
    int rank;
    int world;
    int log_segment;
    const int* pages;
    int pages_per_seq;
};
constexpr int kLogSegmentSmall = 3;        // layers whose prefill launches need their rows' keys split
constexpr int kLogSegmentLarge = 5;        // all others
__host__ __device__ __forceinline__ bool row_is_local(const RowMap& map, int pos) {
    return map.world <= 1 || ((pos / kTileKeys) % map.world) == map.rank;
}
__host__ __device__ __forceinline__ int row_of_position(const RowMap& map, int pos) {
    if (map.world > 1) return ((pos / kTileKeys) / map.world) * kTileKeys + (pos % kTileKeys);
    return map.ring > 0 ? pos % map.ring : pos;
}
// Key tiles are handed out in aligned groups of 2^log_tiles consecutive tiles: the layer's segments
// (log_tiles = map.log_segment) or shorter runs inside them.  group_tiles gives the tiles of one
// group that a block of queries at positions [first_pos, last_pos] attends to on this rank;
// `ordinal` counts from the block's first visible group.  The result is the first tile and the number
// of tiles (`world` apart); a count <= 0 means nothing to do.  Every kernel that produces or merges
// partials derives its work from these functions.
struct TileRange {
    int first;
    int count;
};
__host__ __device__ __forceinline__ int first_visible_tile(int first_pos, int window) {
    return (window > 0 ? (first_pos - window + 1 > 0 ? first_pos - window + 1 : 0) : 0) / kTileKeys;
}
__host__ __device__ __forceinline__ int visible_groups(int first_pos, int last_pos, int window, int log_tiles) {
    return ((last_pos / kTileKeys) >> log_tiles) - (first_visible_tile(first_pos, window) >> log_tiles) + 1;
}
__host__ __device__ __forceinline__ TileRange owned_tiles(const RowMap& map, int t0, int t1) {
    const int world = map.world > 1 ? map.world : 1;
    if (world > 1) t0 += ((map.rank - t0 % world) + world) % world;
    TileRange out;
    out.first = t0;
    out.count = t0 > t1 ? 0 : (t1 - t0) / world + 1;
    return out;
}
__host__ __device__ __forceinline__ TileRange group_tiles(const RowMap& map, int first_pos, int last_pos, int window,
                                                         int ordinal, int log_tiles) {
    const int tile_lo = first_visible_tile(first_pos, window);
    const int tile_hi = last_pos / kTileKeys;
    const int group = (tile_lo >> log_tiles) + ordinal;
    const int g0 = group << log_tiles, g1 = g0 + (1 << log_tiles) - 1;
    return owned_tiles(map, g0 > tile_lo ? g0 : tile_lo, g1 < tile_hi ? g1 : tile_hi);
}
// The tiles of `count` consecutive segments, the first one `first_ordinal` segments after the block's
// first visible segment.
__host__ __device__ __forceinline__ TileRange segment_run_tiles(const RowMap& map, int first_pos, int last_pos, int window,
                                                               int first_ordinal, int count) {
    const int tile_lo = first_visible_tile(first_pos, window);
    const int tile_hi = last_pos / kTileKeys;
    const int segment = (tile_lo >> map.log_segment) + first_ordinal;
    const int g0 = segment << map.log_segment, g1 = ((segment + count) << map.log_segment) - 1;
    return owned_tiles(map, g0 > tile_lo ? g0 : tile_lo, g1 < tile_hi ? g1 : tile_hi);
}
// All the key tiles of this rank that rows at positions first_pos..last_pos see.
__host__ __device__ __forceinline__ TileRange row_tiles(const RowMap& map, int first_pos, int last_pos, int window) {
    return owned_tiles(map, first_visible_tile(first_pos, window), last_pos / kTileKeys);
}

// Where sequence `seq`, kv head `kv_head` keeps position `pos`: the plane of the cache (rows of one
// head) and the row inside it.  Contiguous storage gives every (sequence, head) a plane of its own;
// paged storage one plane per head, shared by the sequences through the page table.
__device__ __forceinline__ int cache_plane(const RowMap& map, int seq, int kv_heads, int kv_head) {
    return map.pages != nullptr ? kv_head : seq * kv_heads + kv_head;
}
__device__ __forceinline__ int cache_row(const RowMap& map, int seq, int pos) {
    if (map.pages != nullptr) {
        return __ldg(map.pages + size_t(seq) * map.pages_per_seq + pos / kTileKeys) * kTileKeys + pos % kTileKeys;
    }
    return row_of_position(map, pos);
}

// First physical row of absolute tile j (callers only ask for tiles they own).
__host__ __device__ __forceinline__ int row_of_tile(const RowMap& map, int tile) {
    return row_of_position(map, tile * kTileKeys);
}

}  // namespace hc
