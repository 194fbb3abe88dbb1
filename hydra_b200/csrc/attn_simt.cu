// attn_simt.cu — the CUDA-core attention kernels: any head_dim up to 512, any group size up to 16.
//
// The kernels share one tile-partial routine (see common.cuh for the canonical computation):
//   decode_runs_kernel    one CTA per (run of key tiles, kv head, sequence): writes the run's tile
//                         partials, or the partial of a whole segment
//   merge_decode_kernel   one CTA per (query head, batch entry): the folds the split kernel left,
//                         then the epilogue (also finishes the decode rows of the tcgen05 kernels)
//   merge_rows_kernel     a warp per (query token, head): the second fold over the segment partials
//                         of a prefill chunk that the tcgen05 kernels split
//   prefill_rows_kernel   one CTA per (kv head, token): both folds in place (with bidirectional
//                         blocks too, like the tcgen05 kernels)
//
// decode = split over key tiles + merge replaces attention_decode / attention_decode_split /
// attention_decode_merge (Sources/HydraMetal/Shaders/attention.metal:132-242, 307-452).
// prefill_rows_kernel replaces attention_prefill (Sources/HydraMetal/Shaders/batch.metal:307-427)
// by the reference's own construction: it is the decode computation with the token index moved
// onto the grid (batch.metal:360-364), which is why it agrees with decode bit for bit.
//
// Unlike the reference's kernels, one CTA serves all the query heads that share a kv head, so each
// K/V byte is read once per group rather than once per query head.
//
// These kernels are the general fallback (and the only path for head_dim 512 or tiny test
// shapes); the tcgen05 kernels in attn_tc.cu serve head_dim 64/128/256.

#include <algorithm>
#include <string>

#include "internal.hpp"

namespace hc {
namespace {

constexpr int kThreads = 128;
constexpr int kSubKeys = 32;                 // keys staged in shared memory at a time
constexpr int kRowPad = 8;                   // bf16 elements of padding per staged row (16 bytes)

struct SimtSmem {
    float* q;        // [G][d]   the group's queries, bf16 values held as float
    float* s;        // [G][128] logits, then weights
    float* acc;      // [G][d]   the tile's O
    float* mm;       // [G]
    float* l;        // [G]
    uint16_t* kv;    // [32][d + 8] staged K or V rows
};

struct FoldState {
    float* A;        // [G][d]
    float* M;        // [G]
    float* L;        // [G]
};

__host__ __device__ inline size_t simt_smem_bytes(int G, int d, int states) {
    size_t floats = size_t(G) * d          // q
                  + size_t(G) * kTileKeys  // s
                  + size_t(G) * d          // acc
                  + 2 * size_t(G);         // mm, l
    floats += size_t(states) * (size_t(G) * d + 2 * size_t(G));   // A, M, L of each fold state
    size_t bytes = floats * 4;
    bytes = (bytes + 15) & ~size_t(15);
    bytes += size_t(kSubKeys) * (d + kRowPad) * 2;
    return bytes;
}

__device__ inline SimtSmem carve(unsigned char* raw, int G, int d, int states, FoldState* state) {
    SimtSmem sm;
    float* f = reinterpret_cast<float*>(raw);
    sm.q = f;            f += size_t(G) * d;
    sm.s = f;            f += size_t(G) * kTileKeys;
    sm.acc = f;          f += size_t(G) * d;
    sm.mm = f;           f += G;
    sm.l = f;            f += G;
    for (int i = 0; i < states; ++i) {
        state[i].A = f;  f += size_t(G) * d;
        state[i].M = f;  f += G;
        state[i].L = f;  f += G;
    }
    size_t offset = size_t(reinterpret_cast<unsigned char*>(f) - raw);
    offset = (offset + 15) & ~size_t(15);
    sm.kv = reinterpret_cast<uint16_t*>(raw + offset);
    return sm;
}

// Copies 32 rows of one head (d bf16 each, contiguous in the cache) into padded shared rows with
// 128-bit loads.
__device__ inline void stage_rows(const uint16_t* __restrict__ rows, uint16_t* dst, int d) {
    const int chunks_per_row = d >> 3;
    const int chunks = kSubKeys * chunks_per_row;
    for (int c = threadIdx.x; c < chunks; c += kThreads) {
        const int row = c / chunks_per_row;
        const int col = c - row * chunks_per_row;
        const uint4 value = *reinterpret_cast<const uint4*>(rows + size_t(row) * d + col * 8);
        *reinterpret_cast<uint4*>(dst + size_t(row) * (d + kRowPad) + col * 8) = value;
    }
}

// The partial of one key tile for the G query rows in sm.q.
//   k_rows, v_rows: the tile's 128 rows of this head in the cache
//   key0: absolute position of the tile's first key; [lo, hi] the visible positions of this query
// Leaves O in sm.acc, mm and l in sm.mm / sm.l.  Ends with a __syncthreads().
__device__ void tile_partial(const SimtSmem& sm, const uint16_t* __restrict__ k_rows,
                             const uint16_t* __restrict__ v_rows, int key0, int lo, int hi, int G,
                             int d, float c) {
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const float neg_inf = __int_as_float(0xff800000);

    // ---- logits: thread (key = lane, heads warp, warp + 4, ...) -------------------------------
    for (int sub = 0; sub < kTileKeys / kSubKeys; ++sub) {
        __syncthreads();                       // previous users of sm.kv are done
        stage_rows(k_rows + size_t(sub) * kSubKeys * d, sm.kv, d);
        __syncthreads();
        const int key = key0 + sub * kSubKeys + lane;
        const bool visible = key >= lo && key <= hi;
        const uint16_t* krow = sm.kv + size_t(lane) * (d + kRowPad);
        for (int g = warp; g < G; g += 4) {
            const float* qrow = sm.q + size_t(g) * d;
            float dot = 0.0f;
            for (int i = 0; i < d; i += 8) {
                const uint4 packed = *reinterpret_cast<const uint4*>(krow + i);
                const float4 qa = *reinterpret_cast<const float4*>(qrow + i);
                const float4 qb = *reinterpret_cast<const float4*>(qrow + i + 4);
                dot = __fmaf_rn(qa.x, __uint_as_float(packed.x << 16), dot);
                dot = __fmaf_rn(qa.y, __uint_as_float(packed.x & 0xffff0000u), dot);
                dot = __fmaf_rn(qa.z, __uint_as_float(packed.y << 16), dot);
                dot = __fmaf_rn(qa.w, __uint_as_float(packed.y & 0xffff0000u), dot);
                dot = __fmaf_rn(qb.x, __uint_as_float(packed.z << 16), dot);
                dot = __fmaf_rn(qb.y, __uint_as_float(packed.z & 0xffff0000u), dot);
                dot = __fmaf_rn(qb.z, __uint_as_float(packed.w << 16), dot);
                dot = __fmaf_rn(qb.w, __uint_as_float(packed.w & 0xffff0000u), dot);
            }
            sm.s[size_t(g) * kTileKeys + sub * kSubKeys + lane] = visible ? dot : neg_inf;
        }
    }
    __syncthreads();

    // ---- per-head maximum, weights and their sum: warp w serves heads w, w + 4, ... ------------
    for (int g = warp; g < G; g += 4) {
        float* srow = sm.s + size_t(g) * kTileKeys;
        float v0 = srow[lane], v1 = srow[lane + 32], v2 = srow[lane + 64], v3 = srow[lane + 96];
        float m = fmaxf(fmaxf(v0, v1), fmaxf(v2, v3));
        #pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, offset));
        }
        const float neg_mc = -__fmul_rn((m == neg_inf) ? 0.0f : m, c);
        v0 = tile_weight(v0, neg_mc, c);
        v1 = tile_weight(v1, neg_mc, c);
        v2 = tile_weight(v2, neg_mc, c);
        v3 = tile_weight(v3, neg_mc, c);
        srow[lane] = v0;
        srow[lane + 32] = v1;
        srow[lane + 64] = v2;
        srow[lane + 96] = v3;
        float sum = __fadd_rn(__fadd_rn(v0, v1), __fadd_rn(v2, v3));
        #pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, offset));
        }
        if (lane == 0) {
            sm.mm[g] = __fmul_rn(m, c);
            sm.l[g] = sum;
        }
    }

    // ---- O = P V: thread owns (head, column pair) items; keys in ascending order ---------------
    const int pairs = d >> 1;
    const int items = G * pairs;
    for (int item = tid; item < items; item += kThreads) {
        sm.acc[size_t(item) * 2] = 0.0f;
        sm.acc[size_t(item) * 2 + 1] = 0.0f;
    }
    for (int sub = 0; sub < kTileKeys / kSubKeys; ++sub) {
        __syncthreads();
        stage_rows(v_rows + size_t(sub) * kSubKeys * d, sm.kv, d);
        __syncthreads();
        for (int item = tid; item < items; item += kThreads) {
            const int g = item / pairs;
            const int cp = item - g * pairs;
            float a0 = sm.acc[size_t(g) * d + 2 * cp];
            float a1 = sm.acc[size_t(g) * d + 2 * cp + 1];
            const float* prow = sm.s + size_t(g) * kTileKeys + sub * kSubKeys;
            #pragma unroll 4
            for (int kk = 0; kk < kSubKeys; kk += 4) {
                const float4 p4 = *reinterpret_cast<const float4*>(prow + kk);
                const float pk[4] = {p4.x, p4.y, p4.z, p4.w};
                #pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t packed = *reinterpret_cast<const uint32_t*>(
                        sm.kv + size_t(kk + u) * (d + kRowPad) + 2 * cp);
                    a0 = __fmaf_rn(pk[u], __uint_as_float(packed << 16), a0);
                    a1 = __fmaf_rn(pk[u], __uint_as_float(packed & 0xffff0000u), a1);
                }
            }
            sm.acc[size_t(g) * d + 2 * cp] = a0;
            sm.acc[size_t(g) * d + 2 * cp + 1] = a1;
        }
    }
    __syncthreads();
}

__device__ inline void load_group_queries(const SimtSmem& sm, const uint16_t* __restrict__ q_row,
                                          int G, int d) {
    // q_row: the G heads of this kv head, contiguous [G][d] bf16.
    for (int i = threadIdx.x; i < G * d; i += kThreads) sm.q[i] = bf16_bits_to_float(q_row[i]);
}

__device__ inline float gate_value(const EpilogueArgs& ep, size_t row, int q_heads, int head, int d,
                                   int i) {
    if (ep.gate_layout == HC_GATE_SEPARATE) {
        return load_io(ep.gate, (row * q_heads + head) * d + i, ep.io_dtype);
    }
    // interleaved: q_proj output [row][head][2d], the gate is the second half of the head's slice
    return load_io(ep.gate, (row * q_heads + head) * size_t(2 * d) + d + i, ep.io_dtype);
}

__device__ inline void write_result(const EpilogueArgs& ep, size_t row, int q_heads, int head, int d,
                                    int i, float A, float M, float L) {
    if (ep.write_partial) {
        float* dst = reinterpret_cast<float*>(ep.out) + (row * q_heads + head) * size_t(d + 2);
        dst[i] = A;
        if (i == 0) {
            dst[d] = M;
            dst[d + 1] = L;
        }
        return;
    }
    const bool gated = ep.gate_layout != HC_GATE_NONE;
    const float g = gated ? gate_value(ep, row, q_heads, head, d, i) : 0.0f;
    store_io(ep.out, (row * q_heads + head) * d + i, ep.io_dtype, finish_value(A, L, gated, g));
}

// ---- the first fold: one segment's tiles into a fold state ---------------------------------------
// Runs tile_partial over the segment's tiles (ascending, `world` apart) and folds each into `st`,
// which starts empty.  Queries of the G heads are in sm.q; [lo, hi] are the visible positions.
__device__ void segment_partial(const SimtSmem& sm, const FoldState& st, const CacheView& cache, int seq, size_t head_rows,
                                const TileRange& tiles, int lo, int hi, int G, int d, float c) {
    for (int i = threadIdx.x; i < G * d; i += kThreads) st.A[i] = 0.0f;
    if (threadIdx.x < G) {
        st.M[threadIdx.x] = kEmptyMax;
        st.L[threadIdx.x] = 0.0f;
    }
    __syncthreads();
    const int world = max(cache.map.world, 1);
    for (int j = 0; j < tiles.count; ++j) {
        const int tile = tiles.first + j * world;
        const size_t row0 = head_rows + cache_row(cache.map, seq, tile * kTileKeys);
        tile_partial(sm, cache.k + row0 * d, cache.v + row0 * d, tile * kTileKeys, lo, hi, G, d, c);
        for (int i = threadIdx.x; i < G * d; i += kThreads) {
            const int g = i / d;
            float Mn, a, b;
            fold_coefficients(st.M[g], sm.mm[g], Mn, a, b);
            st.A[i] = fold_value(st.A[i], a, sm.acc[i], b);
        }
        __syncthreads();
        if (threadIdx.x < G) {
            const int g = threadIdx.x;
            float Mn, a, b;
            fold_coefficients(st.M[g], sm.mm[g], Mn, a, b);
            st.L[g] = __fmaf_rn(st.L[g], a, __fmul_rn(sm.l[g], b));
            st.M[g] = Mn;
        }
        __syncthreads();
    }
}

// ---- decode: one run of key tiles per CTA, its partial(s) to the workspace ---------------------------
// With tile_partials the run's tiles each leave their own partial (slot = ordinal of the tile among the
// row's tiles on this rank); otherwise the run is a whole segment and leaves the segment's partial
// (slot = ordinal of the segment).
__global__ void __launch_bounds__(kThreads)
decode_runs_kernel(const AttnShape shape, const CacheView cache, const BatchMeta meta,
                   const uint16_t* __restrict__ q, float* __restrict__ part_o,
                   float* __restrict__ part_ml, int slots, int log_run, int tile_partials) {
    extern __shared__ __align__(16) unsigned char raw[];
    const int G = shape.group, d = shape.head_dim;
    const int kv_head = blockIdx.y;
    const int b = blockIdx.z;
    const int position = meta.pos[b];
    const TileRange tiles = group_tiles(cache.map, position, position, shape.window, blockIdx.x, log_run);
    if (tiles.count <= 0) return;
    const int lo = shape.window > 0 ? max(0, position - shape.window + 1) : 0;

    FoldState st;
    SimtSmem sm = carve(raw, G, d, 1, &st);
    load_group_queries(sm, q + (size_t(b) * shape.q_heads + size_t(kv_head) * G) * d, G, d);
    const size_t head_rows = size_t(cache_plane(cache.map, meta.seq[b], cache.kv_heads, kv_head)) * cache.capacity;
    const size_t row0 = size_t(b) * shape.q_heads + size_t(kv_head) * G;
    if (tile_partials) {
        const int world = max(cache.map.world, 1);
        const int slot0 = (tiles.first - row_tiles(cache.map, position, position, shape.window).first) / world;
        __syncthreads();
        for (int j = 0; j < tiles.count; ++j) {
            const int tile = tiles.first + j * world;
            const size_t krow = head_rows + cache_row(cache.map, meta.seq[b], tile * kTileKeys);
            tile_partial(sm, cache.k + krow * d, cache.v + krow * d, tile * kTileKeys, lo, position, G, d, shape.c);
            for (int i = threadIdx.x; i < G * d; i += kThreads) {
                const int g = i / d;
                part_o[((row0 + g) * slots + slot0 + j) * d + (i - g * d)] = sm.acc[i];
            }
            if (threadIdx.x < G) {
                part_ml[((row0 + threadIdx.x) * slots + slot0 + j) * 2] = sm.mm[threadIdx.x];
                part_ml[((row0 + threadIdx.x) * slots + slot0 + j) * 2 + 1] = sm.l[threadIdx.x];
            }
            __syncthreads();
        }
        return;
    }
    segment_partial(sm, st, cache, meta.seq[b], head_rows, tiles, lo, position, G, d, shape.c);
    const int slot = blockIdx.x;
    for (int i = threadIdx.x; i < G * d; i += kThreads) {
        const int g = i / d;
        part_o[((row0 + g) * slots + slot) * d + (i - g * d)] = st.A[i];
    }
    if (threadIdx.x < G) {
        part_ml[((row0 + threadIdx.x) * slots + slot) * 2] = st.M[threadIdx.x];
        part_ml[((row0 + threadIdx.x) * slots + slot) * 2 + 1] = st.L[threadIdx.x];
    }
}

// ---- merge for decode rows: both folds over tile partials, or the second over segment partials -------
// One block per (query head, batch entry).  The row's segments are taken sixteen at a time: the
// block's warps first bring each segment's partial into shared memory (folding the segment's tile
// partials, lane l holding columns l, l + 32, ..; or just copying a segment partial), which is where
// a long row's work runs in parallel; then every thread runs the second fold for its columns.
constexpr int kMergeThreads = 256;
constexpr int kMergeSegments = 16;

__host__ __device__ inline size_t merge_smem_bytes(int d) { return size_t(kMergeSegments) * (d + 2) * sizeof(float); }

template <int KCOLS>
__global__ void __launch_bounds__(kMergeThreads)
merge_decode_kernel(const AttnShape shape, const RowMap map, const BatchMeta meta, const float* __restrict__ part_o,
                    const float* __restrict__ part_ml, int slots, int tile_partials, const EpilogueArgs ep) {
    extern __shared__ __align__(16) unsigned char raw[];
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.x;
    const int r = blockIdx.y;
    const int d = shape.head_dim;
    float* seg_o = reinterpret_cast<float*>(raw);                 // [16][d]
    float* seg_ml = seg_o + size_t(kMergeSegments) * d;           // [16][2]; M = -inf marks "nothing here"
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos = meta.pos[r];
    const int world = max(map.world, 1);
    const int ls = map.log_segment;
    const int tile_lo = first_visible_tile(pos, shape.window), tile_hi = pos / kTileKeys;
    const int first_owned = row_tiles(map, pos, pos, shape.window).first;
    const int n_segments = visible_groups(pos, pos, shape.window, ls);
    const int segment0 = tile_lo >> ls;
    const size_t row = size_t(r) * shape.q_heads + head;
    const float neg_inf = __int_as_float(0xff800000);

    float M, L;
    if (shape.count_sink) {
        const uint16_t bits = shape.sinks ? shape.sinks[head] : kNoSinkBits;
        M = __fmul_rn(bf16_bits_to_float(bits), kLog2e);
        L = 1.0f;
    } else {
        M = kEmptyMax;
        L = 0.0f;
    }
    float A[2] = {0.0f, 0.0f};                                    // columns tid and tid + 256

    for (int base = 0; base < n_segments; base += kMergeSegments) {
        const int count = min(kMergeSegments, n_segments - base);
        __syncthreads();
        for (int sl = warp; sl < count; sl += kMergeThreads / 32) {
            const int segment = segment0 + base + sl;
            const int g0 = max(segment << ls, tile_lo), g1 = min((segment << ls) + (1 << ls) - 1, tile_hi);
            const TileRange tiles = owned_tiles(map, g0, g1);
            float m1 = neg_inf, l1 = 0.0f;
            float a1[KCOLS];
            #pragma unroll
            for (int k = 0; k < KCOLS; ++k) a1[k] = 0.0f;
            if (tiles.count > 0 && !tile_partials) {
                const size_t slot = row * slots + base + sl;
                m1 = __ldg(part_ml + slot * 2);
                l1 = __ldg(part_ml + slot * 2 + 1);
                #pragma unroll
                for (int k = 0; k < KCOLS; ++k) {
                    const int col = lane + 32 * k;
                    if (col < d) a1[k] = __ldg(part_o + slot * d + col);
                }
            } else if (tiles.count > 0) {
                // The first fold: the segment's tile partials, ascending, from the empty state.
                m1 = kEmptyMax;
                const size_t slot0 = row * slots + (tiles.first - first_owned) / world;
                constexpr int kAhead = KCOLS <= 4 ? 32 / KCOLS : KCOLS == 8 ? 8 : 4;
                for (int j0 = 0; j0 < tiles.count; j0 += kAhead) {
                    float part[kAhead][KCOLS];
                    float2 ml[kAhead];
                    #pragma unroll
                    for (int u = 0; u < kAhead; ++u) {
                        const bool there = j0 + u < tiles.count;
                        ml[u] = there ? __ldg(reinterpret_cast<const float2*>(part_ml + (slot0 + j0 + u) * 2)) : make_float2(0.0f, 0.0f);
                        #pragma unroll
                        for (int k = 0; k < KCOLS; ++k) {
                            const int col = lane + 32 * k;
                            part[u][k] = (there && col < d) ? __ldg(part_o + (slot0 + j0 + u) * d + col) : 0.0f;
                        }
                    }
                    #pragma unroll
                    for (int u = 0; u < kAhead; ++u) {
                        if (j0 + u < tiles.count) {
                            float Mn, a, b;
                            fold_coefficients(m1, ml[u].x, Mn, a, b);
                            l1 = __fmaf_rn(l1, a, __fmul_rn(ml[u].y, b));
                            m1 = Mn;
                            #pragma unroll
                            for (int k = 0; k < KCOLS; ++k) a1[k] = fold_value(a1[k], a, part[u][k], b);
                        }
                    }
                }
            }
            #pragma unroll
            for (int k = 0; k < KCOLS; ++k) {
                const int col = lane + 32 * k;
                if (col < d) seg_o[size_t(sl) * d + col] = a1[k];
            }
            if (lane == 0) {
                seg_ml[sl * 2] = m1;
                seg_ml[sl * 2 + 1] = l1;
            }
        }
        __syncthreads();
        // The second fold (every thread carries M and L: the same chain, the same bits).
        for (int sl = 0; sl < count; ++sl) {
            const float m1 = seg_ml[sl * 2];
            if (m1 == neg_inf) continue;            // no tile of this segment is on this rank
            float Mn, a, b;
            fold_coefficients(M, m1, Mn, a, b);
            L = __fmaf_rn(L, a, __fmul_rn(seg_ml[sl * 2 + 1], b));
            M = Mn;
            #pragma unroll
            for (int cidx = 0; cidx < 2; ++cidx) {
                const int col = tid + cidx * kMergeThreads;
                if (col < d) A[cidx] = fold_value(A[cidx], a, seg_o[size_t(sl) * d + col], b);
            }
        }
    }
    #pragma unroll
    for (int cidx = 0; cidx < 2; ++cidx) {
        const int col = tid + cidx * kMergeThreads;
        if (col < d) write_result(ep, size_t(r), shape.q_heads, head, d, col, A[cidx], M, L);
    }
}

// ---- merge for many rows of few segments: the second fold over segment partials ----------------------
// Rows are the query tokens of one prefill chunk (row r is the token at first_position + r and shares
// its slots with the other tokens of its 128-row tile) or the entries of a decode batch.
struct MergeRows {
    int decode;              // 1: rows are batch entries at meta.pos[]
    int first_position;      // prefill
    int tokens;              // query tokens, or batch entries
    int tokens_per_tile;     // prefill: 128 / group
    BatchMeta meta;
};

// A warp per row,
// eight rows per block, lane l holding columns (k * 32 + l) * VEC .. + VEC - 1 for k < K.  The
// partials of four segments are fetched before the dependent chain that folds them.
constexpr int kMergeRowsPerBlock = 8;

template <int VEC, int K>
__global__ void __launch_bounds__(kMergeRowsPerBlock * 32)
merge_rows_kernel(const AttnShape shape, const RowMap map, const MergeRows rows, const float* __restrict__ part_o,
                  const float* __restrict__ part_ml, int slots, const EpilogueArgs ep) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const size_t row = size_t(blockIdx.x) * kMergeRowsPerBlock + (threadIdx.x >> 5);    // token * q_heads + head
    if (row >= size_t(rows.tokens) * shape.q_heads) return;
    const int r = int(row / shape.q_heads);
    const int head = int(row - size_t(r) * shape.q_heads);
    const int d = shape.head_dim;
    int first_pos, last_pos;
    if (rows.decode) {
        first_pos = last_pos = rows.meta.pos[r];
    } else {
        const int tile_row0 = (r / rows.tokens_per_tile) * rows.tokens_per_tile;
        first_pos = rows.first_position + tile_row0;
        last_pos = rows.first_position + min(tile_row0 + rows.tokens_per_tile, rows.tokens) - 1;
    }
    const int n_parts = min(visible_groups(first_pos, last_pos, shape.window, map.log_segment), slots);

    float M, L;
    if (shape.count_sink) {
        const uint16_t bits = shape.sinks ? shape.sinks[head] : kNoSinkBits;
        M = __fmul_rn(bf16_bits_to_float(bits), kLog2e);
        L = 1.0f;
    } else {
        M = kEmptyMax;
        L = 0.0f;
    }
    float A[K][VEC];
    #pragma unroll
    for (int k = 0; k < K; ++k) {
        #pragma unroll
        for (int v = 0; v < VEC; ++v) A[k][v] = 0.0f;
    }
    constexpr int kAhead = 4;
    for (int s0 = 0; s0 < n_parts; s0 += kAhead) {
        float part[kAhead][K][VEC];
        float2 ml[kAhead];
        bool present[kAhead];
        #pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const int s = s0 + u;
            // A slot no thread block wrote (this rank owns no tile of that segment) is skipped.
            present[u] = s < n_parts && (map.world <= 1 || group_tiles(map, first_pos, last_pos, shape.window, s, map.log_segment).count > 0);
            ml[u] = make_float2(0.0f, 0.0f);
            if (present[u]) ml[u] = __ldg(reinterpret_cast<const float2*>(part_ml + (row * slots + s) * 2));
            const float* src = part_o + (row * slots + s) * d;
            #pragma unroll
            for (int k = 0; k < K; ++k) {
                const int col = (k * 32 + lane) * VEC;
                if constexpr (VEC == 4) {
                    float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (present[u] && col < d) x = __ldg(reinterpret_cast<const float4*>(src + col));
                    part[u][k][0] = x.x; part[u][k][1] = x.y; part[u][k][2] = x.z; part[u][k][3] = x.w;
                } else if constexpr (VEC == 2) {
                    float2 x = make_float2(0.0f, 0.0f);
                    if (present[u] && col < d) x = __ldg(reinterpret_cast<const float2*>(src + col));
                    part[u][k][0] = x.x; part[u][k][1] = x.y;
                } else {
                    part[u][k][0] = (present[u] && col < d) ? __ldg(src + col) : 0.0f;
                }
            }
        }
        #pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            if (!present[u]) continue;
            float Mn, a, b;
            fold_coefficients(M, ml[u].x, Mn, a, b);
            L = __fmaf_rn(L, a, __fmul_rn(ml[u].y, b));
            M = Mn;
            #pragma unroll
            for (int k = 0; k < K; ++k) {
                #pragma unroll
                for (int v = 0; v < VEC; ++v) A[k][v] = fold_value(A[k][v], a, part[u][k][v], b);
            }
        }
    }
    #pragma unroll
    for (int k = 0; k < K; ++k) {
        #pragma unroll
        for (int v = 0; v < VEC; ++v) {
            const int col = (k * 32 + lane) * VEC + v;
            if (col < d) write_result(ep, size_t(r), shape.q_heads, head, d, col, A[k][v], M, L);
        }
    }
}

// ---- prefill: one (kv head, token) per CTA: the first fold per segment, the second in place -------
__global__ void __launch_bounds__(kThreads)
prefill_rows_kernel(const AttnShape shape, const CacheView cache, int seq,
                    const uint16_t* __restrict__ q, int first_position, const EpilogueArgs ep,
                    const int* __restrict__ block_ends, int appended) {
    extern __shared__ __align__(16) unsigned char raw[];
    const int G = shape.group, d = shape.head_dim;
    const int kv_head = blockIdx.x;
    const int token = blockIdx.y;
    const int position = first_position + token;
    const int lo = shape.window > 0 ? max(0, position - shape.window + 1) : 0;
    // A token of a bidirectional block sees on to the block's end (batch.metal:351-352), as far as
    // keys have been appended.
    int hi = position;
    if (block_ends != nullptr) hi = max(position, min(__ldg(block_ends + token), appended) - 1);

    FoldState st[2];                              // st[0]: the current segment; st[1]: the row
    SimtSmem sm = carve(raw, G, d, 2, st);
    load_group_queries(sm, q + (size_t(token) * shape.q_heads + size_t(kv_head) * G) * d, G, d);
    for (int i = threadIdx.x; i < G * d; i += kThreads) st[1].A[i] = 0.0f;
    if (threadIdx.x < G) {
        if (shape.count_sink) {
            const int head = kv_head * G + threadIdx.x;
            const uint16_t bits = shape.sinks ? shape.sinks[head] : kNoSinkBits;
            st[1].M[threadIdx.x] = __fmul_rn(bf16_bits_to_float(bits), kLog2e);
            st[1].L[threadIdx.x] = 1.0f;
        } else {
            st[1].M[threadIdx.x] = kEmptyMax;
            st[1].L[threadIdx.x] = 0.0f;
        }
    }
    __syncthreads();

    const size_t head_rows = size_t(cache_plane(cache.map, seq, cache.kv_heads, kv_head)) * cache.capacity;
    const int n_slots = visible_groups(position, hi, shape.window, cache.map.log_segment);
    for (int slot = 0; slot < n_slots; ++slot) {
        const TileRange tiles = group_tiles(cache.map, position, hi, shape.window, slot, cache.map.log_segment);
        if (tiles.count <= 0) continue;
        segment_partial(sm, st[0], cache, seq, head_rows, tiles, lo, hi, G, d, shape.c);
        for (int i = threadIdx.x; i < G * d; i += kThreads) {
            const int g = i / d;
            float Mn, a, b;
            fold_coefficients(st[1].M[g], st[0].M[g], Mn, a, b);
            st[1].A[i] = fold_value(st[1].A[i], a, st[0].A[i], b);
        }
        __syncthreads();
        if (threadIdx.x < G) {
            const int g = threadIdx.x;
            float Mn, a, b;
            fold_coefficients(st[1].M[g], st[0].M[g], Mn, a, b);
            st[1].L[g] = __fmaf_rn(st[1].L[g], a, __fmul_rn(st[0].L[g], b));
            st[1].M[g] = Mn;
        }
        __syncthreads();
    }

    for (int i = threadIdx.x; i < G * d; i += kThreads) {
        const int g = i / d;
        write_result(ep, size_t(token), shape.q_heads, kv_head * G + g, d, i - g * d, st[1].A[i], st[1].M[g], st[1].L[g]);
    }
}

// ---- combine: the fold over ranks of a sequence-sharded cache ----------------------------------
__global__ void combine_ranks_kernel(const float* __restrict__ gathered, int world, int rows,
                                     int q_heads, int d, const EpilogueArgs ep) {
    const size_t vec = blockIdx.x;                 // row * q_heads + head
    const size_t row = vec / q_heads;
    const int head = int(vec % q_heads);
    const size_t stride = size_t(rows) * q_heads * (d + 2);
    const float* p0 = gathered + vec * (d + 2);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float M = p0[d], L = p0[d + 1], A = p0[i];
        for (int r = 1; r < world; ++r) {
            const float* pr = p0 + size_t(r) * stride;
            float Mn, a, b;
            fold_coefficients(M, pr[d], Mn, a, b);
            L = __fmaf_rn(L, a, __fmul_rn(pr[d + 1], b));
            A = fold_value(A, a, pr[i], b);
            M = Mn;
        }
        const bool gated = ep.gate_layout != HC_GATE_NONE;
        const float g = gated ? gate_value(ep, row, q_heads, head, d, i) : 0.0f;
        store_io(ep.out, vec * d + i, ep.io_dtype, finish_value(A, L, gated, g));
    }
}

}  // namespace

hc_status simt_prefill(hc_context* ctx, const AttnShape& shape, const CacheView& cache, int seq,
                       const uint16_t* q, int tokens, int first_position, const EpilogueArgs& ep,
                       cudaStream_t stream, const int* block_ends) {
    if (tokens <= 0) return HC_OK;
    const size_t smem = simt_smem_bytes(shape.group, shape.head_dim, 2);
    cudaError_t err = cudaFuncSetAttribute(prefill_rows_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (err != cudaSuccess) return check_cuda(err, "prefill_rows_kernel shared memory");
    for (int start = 0; start < tokens; start += 32768) {
        const int count = tokens - start < 32768 ? tokens - start : 32768;
        EpilogueArgs sub = ep;
        if (start > 0) {
            // Offsets are in rows; the epilogue indexes rows from its base pointer.
            const size_t out_row = ep.write_partial ? size_t(shape.q_heads) * (shape.head_dim + 2) * 4
                                 : size_t(shape.q_heads) * shape.head_dim * (ep.io_dtype == HC_F32 ? 4 : 2);
            sub.out = static_cast<unsigned char*>(ep.out) + size_t(start) * out_row;
            if (ep.gate_layout != HC_GATE_NONE) {
                const size_t mult = ep.gate_layout == HC_GATE_INTERLEAVED ? 2 : 1;
                const size_t gate_row = size_t(shape.q_heads) * shape.head_dim * mult
                                      * (ep.io_dtype == HC_F32 ? 4 : 2);
                sub.gate = static_cast<const unsigned char*>(ep.gate) + size_t(start) * gate_row;
            }
        }
        dim3 grid(shape.kv_heads, count);
        prefill_rows_kernel<<<grid, kThreads, smem, stream>>>(
            shape, cache, seq, q + size_t(start) * shape.q_heads * shape.head_dim,
            first_position + start, sub, block_ends ? block_ends + start : nullptr, first_position + tokens);
        ctx->launches += 1;
        err = cudaGetLastError();
        if (err != cudaSuccess) return check_cuda(err, "prefill_rows_kernel launch");
    }
    return HC_OK;
}

DecodePlan plan_decode(const AttnShape& shape, const RowMap& map, const BatchMeta& meta, int n_seq, int target_items,
                       bool allow_whole, int max_run_segments) {
    DecodePlan plan{};
    int most_tiles = 0, segments = 0, most_segments = 1;
    for (int b = 0; b < n_seq; ++b) {
        most_tiles = std::max(most_tiles, row_tiles(map, meta.pos[b], meta.pos[b], shape.window).count);
        const int n = visible_groups(meta.pos[b], meta.pos[b], shape.window, map.log_segment);
        segments += n;
        most_segments = std::max(most_segments, n);
    }
    plan.tiles = std::max(most_tiles, 1);
    plan.log_run = map.log_segment;
    plan.run_segments = 1;
    // The coarsest cut that still gives the machine enough items: whole rows, then runs of segments,
    // then shorter and shorter runs of tiles.  Rows of a tile or two are never cut: the merge would
    // cost more than it saves.
    if (allow_whole && (most_tiles <= 2 || n_seq * shape.kv_heads >= target_items)) {
        plan.finish = 1;
        plan.slots = 1;
        return plan;
    }
    if (segments * shape.kv_heads >= target_items) {
        plan.run_segments = std::max(1, std::min(max_run_segments, segments * shape.kv_heads / target_items));
        plan.slots = most_segments;
        return plan;
    }
    int log_run = map.log_segment - 1;
    for (; log_run > 0; --log_run) {
        int items = 0;
        for (int b = 0; b < n_seq; ++b) items += visible_groups(meta.pos[b], meta.pos[b], shape.window, log_run);
        if (items * shape.kv_heads >= target_items) break;
    }
    plan.log_run = log_run;
    plan.tile_partials = 1;
    plan.slots = plan.tiles;
    return plan;
}

DecodePlan simt_plan_decode(const hc_context* ctx, const AttnShape& shape, const RowMap& map, const BatchMeta& meta, int n_seq) {
    // These kernels always leave partials and merge: a whole-row plan is run as whole segments.
    DecodePlan plan = plan_decode(shape, map, meta, n_seq, 4 * ctx->sm_count, true, 1);
    if (plan.finish) {
        plan.finish = 0;
        plan.tile_partials = 0;
        plan.log_run = map.log_segment;
        plan.slots = 1;
        for (int b = 0; b < n_seq; ++b) {
            plan.slots = std::max(plan.slots, visible_groups(meta.pos[b], meta.pos[b], shape.window, map.log_segment));
        }
    }
    return plan;
}

hc_status simt_decode(hc_context* ctx, const AttnShape& shape, const CacheView& cache,
                      const BatchMeta& meta, int n_seq, const uint16_t* q, const Workspace& ws,
                      const EpilogueArgs& ep, cudaStream_t stream) {
    if (n_seq <= 0) return HC_OK;
    const DecodePlan plan = simt_plan_decode(ctx, shape, cache.map, meta, n_seq);
    const size_t rows = size_t(n_seq) * shape.q_heads;
    if (rows * plan.slots * shape.head_dim > ws.part_o_floats || rows * plan.slots * 2 > ws.part_ml_floats) {
        return fail(HC_KV_OVERFLOW, "decode: the split-attention workspace is too small for this call");
    }
    int runs = 1;
    for (int b = 0; b < n_seq; ++b) runs = std::max(runs, visible_groups(meta.pos[b], meta.pos[b], shape.window, plan.log_run));
    const size_t smem = simt_smem_bytes(shape.group, shape.head_dim, 1);
    cudaError_t err = cudaFuncSetAttribute(decode_runs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (err != cudaSuccess) return check_cuda(err, "decode_runs_kernel shared memory");
    dim3 grid(runs, shape.kv_heads, n_seq);
    decode_runs_kernel<<<grid, kThreads, smem, stream>>>(shape, cache, meta, q, ws.part_o, ws.part_ml, plan.slots,
                                                         plan.log_run, plan.tile_partials);
    ctx->launches += 1;
    err = cudaGetLastError();
    if (err != cudaSuccess) return check_cuda(err, "decode_runs_kernel launch");
    return launch_merge_decode(ctx, shape, cache.map, meta, n_seq, ws, plan, ep, stream);
}

static hc_status launch_merge_rows(hc_context* ctx, const AttnShape& shape, const RowMap& map, const MergeRows& rows,
                                   const Workspace& ws, int slots, const EpilogueArgs& ep, cudaStream_t stream) {
    const int d = shape.head_dim;
    auto kernel = d == 64 ? merge_rows_kernel<2, 1> : d == 128 ? merge_rows_kernel<4, 1> : d == 256 ? merge_rows_kernel<4, 2>
                : d == 512 ? merge_rows_kernel<4, 4> : merge_rows_kernel<1, 16>;
    const size_t n_rows = size_t(rows.tokens) * shape.q_heads;
    const unsigned blocks = unsigned((n_rows + kMergeRowsPerBlock - 1) / kMergeRowsPerBlock);
    const cudaError_t launched = launch_pdl(kernel, dim3(blocks), dim3(kMergeRowsPerBlock * 32), 0, stream, shape, map, rows,
                                            static_cast<const float*>(ws.part_o), static_cast<const float*>(ws.part_ml),
                                            slots, ep);
    ctx->launches += 1;
    if (launched != cudaSuccess) return check_cuda(launched, "merge_rows_kernel launch");
    return check_cuda(cudaGetLastError(), "merge_rows_kernel launch");
}

hc_status launch_merge_decode(hc_context* ctx, const AttnShape& shape, const RowMap& map, const BatchMeta& meta, int n_seq,
                              const Workspace& ws, const DecodePlan& plan, const EpilogueArgs& ep, cudaStream_t stream) {
    if (!plan.tile_partials && (plan.slots <= 8 || n_seq * shape.q_heads >= 1024)) {
        // Few segment partials a row, or rows enough to fill the machine with one warp each: a warp per
        // row does it without the staging below.
        MergeRows rows{};
        rows.decode = 1;
        rows.tokens = n_seq;
        rows.meta = meta;
        return launch_merge_rows(ctx, shape, map, rows, ws, plan.slots, ep, stream);
    }
    const int d = shape.head_dim;
    const int kcols = (d + 31) / 32;
    auto kernel = kcols <= 2 ? merge_decode_kernel<2> : kcols <= 4 ? merge_decode_kernel<4>
                : kcols <= 8 ? merge_decode_kernel<8> : merge_decode_kernel<16>;
    const cudaError_t launched = launch_pdl(kernel, dim3(shape.q_heads, n_seq), dim3(kMergeThreads), merge_smem_bytes(d), stream,
                                            shape, map, meta, static_cast<const float*>(ws.part_o),
                                            static_cast<const float*>(ws.part_ml), plan.slots, plan.tile_partials, ep);
    ctx->launches += 1;
    if (launched != cudaSuccess) return check_cuda(launched, "merge_decode_kernel launch");
    return check_cuda(cudaGetLastError(), "merge_decode_kernel launch");
}

hc_status launch_merge_prefill(hc_context* ctx, const AttnShape& shape, const RowMap& map, int tokens, int first_position,
                               const Workspace& ws, int slots, const EpilogueArgs& ep, cudaStream_t stream) {
    MergeRows rows{};
    rows.first_position = first_position;
    rows.tokens = tokens;
    rows.tokens_per_tile = kTileKeys / shape.group;        // a row tile is 128 rows: 128 / group tokens
    return launch_merge_rows(ctx, shape, map, rows, ws, slots, ep, stream);
}

hc_status launch_combine(hc_context* ctx, const float* gathered, int world, int rows, int q_heads,
                         int d, const EpilogueArgs& ep, cudaStream_t stream) {
    if (rows <= 0) return HC_OK;
    combine_ranks_kernel<<<unsigned(size_t(rows) * q_heads), 128, 0, stream>>>(gathered, world, rows,
                                                                               q_heads, d, ep);
    ctx->launches += 1;
    return check_cuda(cudaGetLastError(), "combine_ranks_kernel launch");
}

// ---- decode without any allocation ----------------------------------------------------------------
//
// Some hosts cannot allocate device memory at the moment they need attention: a runner that has
// handed every byte of the device to its weight and KV pools, a plugin loaded into a process whose
// allocator it must not touch, or a caller inside a region where cudaMalloc is forbidden.  For
// them the split-decode partials live in this fixed array instead of a workspace that
// hc_kv_cache_create would size.  Every GPU that loads the library holds these 8 MiB until the
// process exits.
constexpr size_t kStaticScratchFloats = size_t(2) << 20;               // 8 MiB
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

// `g_static_scratch` in host code is only a handle, not a device address: a kernel given it would
// fault or, where the GPU can reach host memory, quietly use the wrong memory.  The device address
// comes from cudaGetSymbolAddress, asked at context creation with that device current.
hc_status static_scratch_prepare(int device, float** address) {
    *address = nullptr;
    int current = -1;
    cudaError_t err = cudaGetDevice(&current);
    if (err == cudaSuccess && current != device) {
        return fail(HC_INVALID_ARGUMENT, "static scratch: device " + std::to_string(device) + " is not current");
    }
    void* ptr = nullptr;
    if (err == cudaSuccess) err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess || !ptr) {
        return check_cuda(err == cudaSuccess ? cudaErrorInvalidSymbol : err, "address of the static decode scratch");
    }
    *address = static_cast<float*>(ptr);
    return HC_OK;
}

hc_status static_decode_inputs(hc_context* ctx, hc_kv_cache* cache, int layer, const int* seq_ids,
                               const int* positions, int n_seq, const void* q, void* out,
                               const hc_attn_params* p, AttnShape* shape, CacheView* view, BatchMeta* meta,
                               EpilogueArgs* ep, const hc_layer_store** store, bool* tensor);

}  // namespace hc

extern "C" {

size_t hc_attention_decode_static_limit(void) { return hc::kStaticScratchFloats * sizeof(float); }

hc_status hc_attention_decode_static(hc_context* ctx, hc_kv_cache* cache, int layer, const int* seq_ids,
                                     const int* positions, int n_seq, const void* q, void* out,
                                     const hc_attn_params* params, void* stream) {
    using namespace hc;
    AttnShape shape{};
    CacheView view{};
    BatchMeta meta{};
    EpilogueArgs ep{};
    const hc_layer_store* store = nullptr;
    bool tensor = false;
    hc_status st = static_decode_inputs(ctx, cache, layer, seq_ids, positions, n_seq, q, out, params, &shape,
                                        &view, &meta, &ep, &store, &tensor);
    if (st != HC_OK) return st;
    if (!ctx->static_scratch) return fail(HC_CUDA_ERROR, "this context has no static scratch address");
    // The cut the default path would make (given this much room), and its partials: [rows][slots][2]
    // first, then [rows][slots][d].  A whole-row cut leaves no partials; the tensor-core kernels then
    // keep their second-fold state, if any, where the partials would be.
    const DecodePlan plan = tensor ? tc_plan_decode(ctx, shape, view.map, meta, n_seq, kStaticScratchFloats)
                                   : simt_plan_decode(ctx, shape, view.map, meta, n_seq);
    const size_t rows = size_t(n_seq) * shape.q_heads;
    const size_t ml_floats = plan.finish ? 0 : (rows * plan.slots * 2 + 3) & ~size_t(3);
    const size_t need = plan.finish ? 0 : ml_floats + rows * plan.slots * shape.head_dim;
    if (need > kStaticScratchFloats) {
        return fail(HC_KV_OVERFLOW, "hc_attention_decode_static: this call needs " + std::to_string(need * 4) +
                                        " bytes of partials, the fixed scratch holds " +
                                        std::to_string(kStaticScratchFloats * 4));
    }
    // Every partial the merge reads is written by this call's split kernel first, so nothing in the
    // array has to start at zero.
    Workspace ws;
    ws.part_ml = ctx->static_scratch;
    ws.part_ml_floats = ml_floats;
    ws.part_o = ctx->static_scratch + ml_floats;
    ws.part_o_floats = kStaticScratchFloats - ml_floats;
    // The same kernels, in the same order, as hc_attention_decode: only the partials live elsewhere,
    // so the two entry points return the same bits.
    if (tensor) {
        return tc_decode(ctx, shape, *store, view, meta, n_seq, static_cast<const uint16_t*>(q), ws, ep,
                         static_cast<cudaStream_t>(stream));
    }
    return simt_decode(ctx, shape, view, meta, n_seq, static_cast<const uint16_t*>(q), ws, ep,
                       static_cast<cudaStream_t>(stream));
}

}  // extern "C"
