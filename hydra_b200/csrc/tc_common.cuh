// tc_common.cuh — what the tcgen05 attention kernels share: the kernel arguments, the work-item list a
// persistent CTA walks, and small helpers.
#pragma once

#include "internal.hpp"
#include "tc_ptx.cuh"

namespace hc {
namespace {

struct TcArgs {
    const uint16_t* q;        // bf16 [rows][q_heads][d], prepared
    int tokens;               // prefill: tokens of the chunk; decode: batch entries
    int first_position;
    int q_heads;
    int kv_heads;
    int log_group;
    int window;
    float c;
    const uint16_t* sinks;
    int count_sink;
    int seq;
    RowMap map;
    EpilogueArgs ep;
    int* status;
    int n_items;              // work items in the list
    int mtiles;               // prefill: row tiles per kv head
    // How a launch cuts its rows' keys into items (the bits are the same whichever the host picks):
    //   finish != 0       an item is all the key tiles of one row tile and kv head (prefill) or of one
    //                     sequence and kv head (decode).  The kernel runs both folds and the epilogue,
    //                     keeping the second fold's values between segments in row_state.
    //   otherwise         the kernel writes partials to the workspace, `slots` per row at most, and a
    //                     merge kernel finishes the rows.  With tile_partials == 0 an item is a run of
    //                     whole segments (one in prefill; seq_run[b] in decode, so that a sequence's
    //                     items are of one size) and leaves each segment's partial, slot = ordinal of
    //                     the segment.  With tile_partials != 0 (decode only) an item is an aligned run
    //                     of 2^log_run tiles, log_run < map.log_segment, and leaves every tile's own
    //                     partial, slot = ordinal of the tile among the row's tiles.
    int decode;
    int slots;
    int finish;
    int log_run;
    int tile_partials;
    float* part_o;            // fp32 [rows][slots][d]
    float* part_ml;           // fp32 [rows][slots][2]
    float* row_state;         // fp32 [thread blocks][d][128], finish only
    // Multipliers for the divisions of decode_item (see fast_div); 0 = divide the ordinary way.
    uint32_t magic_slots, magic_kv_heads;
    // Decode: sequence b has seq_slots[b] runs; its items, kv head major, start at item_start[b].
    int item_start[kMaxBatch + 1];
    unsigned short seq_slots[kMaxBatch];
    unsigned short seq_run[kMaxBatch];   // segments per run of sequence b (decode, segment partials)
    uint32_t seq_magic[kMaxBatch];       // division by seq_slots[b]
    BatchMeta meta;
    // Prefill with bidirectional blocks: per token of the call, one past the end of its block (0 =
    // none), and the position one past the last key appended.  Every item then reaches to the last
    // appended key's tile; rows that see nothing of a tile fold its empty partial, a no-op.
    const int* block_ends;
    int appended;
};

// n / d for the small operands of the item list: with magic = ceil(2^32 / d) the high word of
// n * magic is the quotient whenever n * d < 2^32, which the host checks before it sets a magic.
__host__ __device__ inline uint32_t division_magic(uint32_t d, uint32_t n_max) {
    if (d <= 1 || uint64_t(n_max) * d >= (1ull << 32)) return 0;
    return uint32_t(((1ull << 32) + d - 1) / d);
}
__device__ __forceinline__ int fast_div(int n, int d, uint32_t magic) {
    return magic != 0 ? int(__umulhi(uint32_t(n), magic)) : n / d;
}


struct TcItem {
    int kv_head;
    int seq;
    int row0;          // first row of q / out (token index of the chunk, or batch entry)
    int valid_tokens;  // query tokens in this row tile
    int first_pos;     // position of the first query token
    int tile_first;    // absolute index of the first key tile
    int n_tiles;       // key tiles to visit (stride `world` apart); <= 0: nothing to do
    int slot;          // ordinal of the item's run among the rows' runs; with tile partials, the row's
                       // partial slot of the item's first tile
    int first_segment; // absolute index of the first segment the rows see (segment partials go to
                       // slot = segment - first_segment)
};

__device__ __forceinline__ TcItem decode_item(const TcArgs& args, int index) {
    TcItem w;
    const int tokens_per_tile = kRows >> args.log_group;
    if (args.decode) {
        int lo = 0, hi = args.tokens;                 // item_start[lo] <= index < item_start[hi]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (index >= args.item_start[mid]) lo = mid; else hi = mid;
        }
        const int b = lo;
        const int local = index - args.item_start[b];
        const int slots = args.seq_slots[b];
        w.kv_head = fast_div(local, slots, args.seq_magic[b]);
        w.slot = local - w.kv_head * slots;
        w.row0 = b;
        w.valid_tokens = 1;
        w.first_pos = args.meta.pos[b];
        w.seq = args.meta.seq[b];
    } else {
        // Longest key ranges first: descending row tile; a row tile's segments and kv heads adjacent.
        const int rest = fast_div(index, args.slots, args.magic_slots);
        w.slot = index - rest * args.slots;
        const int tile_index = fast_div(rest, args.kv_heads, args.magic_kv_heads);
        w.kv_head = rest - tile_index * args.kv_heads;
        const int mtile = args.mtiles - 1 - tile_index;
        w.row0 = mtile * tokens_per_tile;
        w.valid_tokens = min(tokens_per_tile, args.tokens - w.row0);
        w.first_pos = args.first_position + w.row0;
        w.seq = args.seq;
    }
    const int last_pos = (!args.decode && args.block_ends != nullptr) ? args.appended - 1 : w.first_pos + w.valid_tokens - 1;
    TileRange tiles;
    if (args.finish) {
        tiles = row_tiles(args.map, w.first_pos, last_pos, args.window);
    } else if (args.decode && !args.tile_partials) {
        const int run = args.seq_run[w.row0];           // the sequence's segments in runs of one size
        tiles = segment_run_tiles(args.map, w.first_pos, last_pos, args.window, w.slot * run, run);
    } else {
        tiles = group_tiles(args.map, w.first_pos, last_pos, args.window, w.slot, args.log_run);
    }
    w.tile_first = tiles.first;
    w.n_tiles = tiles.count;
    w.first_segment = first_visible_tile(w.first_pos, args.window) >> args.map.log_segment;
    if (args.tile_partials && tiles.count > 0) {
        const int world = args.map.world > 1 ? args.map.world : 1;
        w.slot = (tiles.first - row_tiles(args.map, w.first_pos, last_pos, args.window).first) / world;
    }
    return w;
}

// The walk over a CTA's items: each item is decoded once per role (its decoding costs a few integer
// divisions, which a role pays on its critical path at every item boundary).
struct TcItemIter {
    int item;          // index in the work list, or n_items at the end
    TcItem w;
};
__device__ __forceinline__ void items_seek(const TcArgs& args, TcItemIter& it) {
    for (; it.item < args.n_items; it.item += gridDim.x) {
        it.w = decode_item(args, it.item);
        if (it.w.n_tiles > 0) return;
    }
    it.item = args.n_items;
}
__device__ __forceinline__ TcItemIter items_begin(const TcArgs& args) {
    TcItemIter it;
    it.item = blockIdx.x;
    it.w = TcItem{};
    items_seek(args, it);
    return it;
}
__device__ __forceinline__ void items_next(const TcArgs& args, TcItemIter& it) {
    it.item += gridDim.x;
    items_seek(args, it);
}

// bf16x2 of two softmax weights: `lo` in the low half (the earlier key), `hi` in the high half.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t packed;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
    return packed;
}


// (x0, x1) <- (x0 * c + d, x1 * c + d), each rounded once, as one packed instruction.
__device__ __forceinline__ void fma2_inplace(uint32_t& x0, uint32_t& x1, float c, float d) {
    uint64_t x = uint64_t(x0) | (uint64_t(x1) << 32);
    const uint64_t cc = uint64_t(__float_as_uint(c)) | (uint64_t(__float_as_uint(c)) << 32);
    const uint64_t dd = uint64_t(__float_as_uint(d)) | (uint64_t(__float_as_uint(d)) << 32);
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(x) : "l"(x), "l"(cc), "l"(dd));
    x0 = uint32_t(x);
    x1 = uint32_t(x >> 32);
}

// Two steps of the fold at once: (A0, A1) <- (A0 * a + (o0 * b), A1 * a + (o1 * b)), every product
// and sum rounded exactly as fold_value does, in two packed instructions instead of four.
__device__ __forceinline__ void fold_value2(float& A0, float& A1, float a, uint32_t o0, uint32_t o1, float b) {
    uint64_t acc = uint64_t(__float_as_uint(A0)) | (uint64_t(__float_as_uint(A1)) << 32);
    const uint64_t o = uint64_t(o0) | (uint64_t(o1) << 32);
    const uint64_t aa = uint64_t(__float_as_uint(a)) | (uint64_t(__float_as_uint(a)) << 32);
    const uint64_t bb = uint64_t(__float_as_uint(b)) | (uint64_t(__float_as_uint(b)) << 32);
    uint64_t ob;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(ob) : "l"(o), "l"(bb));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(acc) : "l"(acc), "l"(aa), "l"(ob));
    A0 = __uint_as_float(uint32_t(acc));
    A1 = __uint_as_float(uint32_t(acc >> 32));
}

}  // namespace
}  // namespace hc
