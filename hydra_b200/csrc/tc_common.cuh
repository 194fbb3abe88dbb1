// tc_common.cuh — what the tcgen05 attention kernels share: the kernel arguments, the work-item list a
// persistent CTA walks, and small helpers.
#pragma once

#include "internal.hpp"
#include "tc_ptx.cuh"

namespace hc {
namespace {

struct TcArgs {
    const uint16_t* q;        // bf16 [rows][q_heads][d], prepared
    int tokens;               // prefill: tokens of the chunk
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
    // Decode (split over key tiles): one query token per batch entry; an item is a run of
    // `tiles_per_item` consecutive key tiles of one (sequence, kv head) whose partials it writes.
    int decode;
    int chunks;               // decode: items per (sequence, kv head)
    int tiles_per_item;
    float* part_o;            // fp32 [rows][part_tiles][d]
    float* part_ml;           // fp32 [rows][part_tiles][2]
    int part_tiles;
    // Multipliers for the divisions of decode_item (see fast_div); 0 = divide the ordinary way.
    uint32_t magic_chunks, magic_kv_heads, magic_world;
    // Decode, per-sequence item lists (per_seq != 0; used when the cache is not sequence-sharded):
    // sequence b's key tiles are cut into seq_chunks[b] runs of seq_tiles[b] tiles (the last one may
    // be shorter, never empty), so ragged batches leave no empty items and the runs of one sequence
    // are of one size.  Its items, kv head major, start at item_start[b].
    int per_seq;
    int item_start[kMaxBatch + 1];
    unsigned short seq_chunks[kMaxBatch];
    unsigned short seq_tiles[kMaxBatch];
    uint32_t seq_magic[kMaxBatch];       // division by seq_chunks[b]
    BatchMeta meta;
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
    int ordinal0;      // decode: ordinal of the first tile among the row's tiles
};

__device__ __forceinline__ TcItem decode_item(const TcArgs& args, int index) {
    TcItem w;
    const int tokens_per_tile = kRows >> args.log_group;
    int chunk = 0;
    int tiles_per_item = args.tiles_per_item;
    if (args.decode) {
        int b;
        if (args.per_seq) {
            int lo = 0, hi = args.tokens;                 // item_start[lo] <= index < item_start[hi]
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (index >= args.item_start[mid]) lo = mid; else hi = mid;
            }
            b = lo;
            const int local = index - args.item_start[b];
            const int chunks = args.seq_chunks[b];
            w.kv_head = fast_div(local, chunks, args.seq_magic[b]);
            chunk = local - w.kv_head * chunks;
            tiles_per_item = args.seq_tiles[b];
        } else {
            const int rest = fast_div(index, args.chunks, args.magic_chunks);
            chunk = index - rest * args.chunks;
            b = fast_div(rest, args.kv_heads, args.magic_kv_heads);
            w.kv_head = rest - b * args.kv_heads;
        }
        w.row0 = b;
        w.valid_tokens = 1;
        w.first_pos = args.meta.pos[b];
        w.seq = args.meta.seq[b];
    } else {
        // Longest key ranges first: descending row tile, the kv heads of one row tile adjacent.
        const int tile_index = fast_div(index, args.kv_heads, args.magic_kv_heads);
        w.kv_head = index - tile_index * args.kv_heads;
        const int mtile = args.mtiles - 1 - tile_index;
        w.row0 = mtile * tokens_per_tile;
        w.valid_tokens = min(tokens_per_tile, args.tokens - w.row0);
        w.first_pos = args.first_position + w.row0;
        w.seq = args.seq;
    }
    const int last_pos = w.first_pos + w.valid_tokens - 1;
    const int lo_first = args.window > 0 ? max(0, w.first_pos - args.window + 1) : 0;
    const int world = max(args.map.world, 1);
    int tile_first = lo_first / kTileKeys;
    const int tile_last = last_pos / kTileKeys;
    if (world > 1) tile_first += ((args.map.rank - tile_first % world) + world) % world;
    int n_tiles = tile_first > tile_last ? 0
                  : (world > 1 ? fast_div(tile_last - tile_first, world, args.magic_world) : tile_last - tile_first) + 1;
    w.ordinal0 = 0;
    if (args.decode) {
        w.ordinal0 = chunk * tiles_per_item;
        tile_first += w.ordinal0 * world;
        n_tiles = min(tiles_per_item, n_tiles - w.ordinal0);
    }
    w.tile_first = tile_first;
    w.n_tiles = n_tiles;
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
