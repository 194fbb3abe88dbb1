// attn_simt.cu — the CUDA-core attention kernels: any head_dim up to 512, any group size up to 16.
//
// Three kernels share one tile-partial routine (see common.cuh for the canonical computation):
//   decode_tiles_kernel   one CTA per (key tile, kv head, sequence): writes the tile's partial
//   merge_tiles_kernel    one CTA per (query head, sequence): folds the partials in tile order
//   prefill_rows_kernel   one CTA per (kv head, token): walks the token's tiles and folds in place
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

__host__ __device__ inline size_t simt_smem_bytes(int G, int d, bool with_state) {
    size_t floats = size_t(G) * d          // q
                  + size_t(G) * kTileKeys  // s
                  + size_t(G) * d          // acc
                  + 2 * size_t(G);         // mm, l
    if (with_state) floats += size_t(G) * d + 2 * size_t(G);   // A, M, L
    size_t bytes = floats * 4;
    bytes = (bytes + 15) & ~size_t(15);
    bytes += size_t(kSubKeys) * (d + kRowPad) * 2;
    return bytes;
}

__device__ inline SimtSmem carve(unsigned char* raw, int G, int d, bool with_state, float** A,
                                 float** M, float** L) {
    SimtSmem sm;
    float* f = reinterpret_cast<float*>(raw);
    sm.q = f;            f += size_t(G) * d;
    sm.s = f;            f += size_t(G) * kTileKeys;
    sm.acc = f;          f += size_t(G) * d;
    sm.mm = f;           f += G;
    sm.l = f;            f += G;
    if (with_state) {
        *A = f;          f += size_t(G) * d;
        *M = f;          f += G;
        *L = f;          f += G;
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

// First and last absolute tile a query at `position` touches, restricted to tiles this rank owns.
__device__ __host__ inline void tile_span(int position, int window, int& lo, int& first_tile,
                                          int& last_tile) {
    lo = window > 0 ? max(0, position - window + 1) : 0;
    first_tile = lo / kTileKeys;
    last_tile = position / kTileKeys;
}

// ---- decode: one tile per CTA -----------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
decode_tiles_kernel(const AttnShape shape, const CacheView cache, const BatchMeta meta,
                    const uint16_t* __restrict__ q, float* __restrict__ part_o,
                    float* __restrict__ part_ml, int part_tiles) {
    extern __shared__ __align__(16) unsigned char raw[];
    const int G = shape.group, d = shape.head_dim;
    const int kv_head = blockIdx.y;
    const int b = blockIdx.z;
    const int position = meta.pos[b];
    int lo, first_tile, last_tile;
    tile_span(position, shape.window, lo, first_tile, last_tile);
    // Local tiles: with a sequence-sharded cache this rank owns tiles congruent to rank mod world.
    const int world = max(cache.map.world, 1);
    int tile = first_tile + blockIdx.x;
    if (world > 1) {
        const int first_owned = first_tile + ((cache.map.rank - first_tile % world) + world) % world;
        tile = first_owned + blockIdx.x * world;
    }
    if (tile > last_tile) return;

    SimtSmem sm = carve(raw, G, d, false, nullptr, nullptr, nullptr);
    load_group_queries(sm, q + (size_t(b) * shape.q_heads + size_t(kv_head) * G) * d, G, d);
    const size_t head_rows = (size_t(meta.seq[b]) * cache.kv_heads + kv_head) * cache.capacity;
    const size_t row0 = head_rows + row_of_tile(cache.map, tile);
    tile_partial(sm, cache.k + row0 * d, cache.v + row0 * d, tile * kTileKeys, lo, position, G, d,
                 shape.c);

    for (int i = threadIdx.x; i < G * d; i += kThreads) {
        const int g = i / d;
        const size_t row = size_t(b) * shape.q_heads + size_t(kv_head) * G + g;
        part_o[(row * part_tiles + blockIdx.x) * d + (i - g * d)] = sm.acc[i];
    }
    if (threadIdx.x < G) {
        const size_t row = size_t(b) * shape.q_heads + size_t(kv_head) * G + threadIdx.x;
        part_ml[(row * part_tiles + blockIdx.x) * 2] = sm.mm[threadIdx.x];
        part_ml[(row * part_tiles + blockIdx.x) * 2 + 1] = sm.l[threadIdx.x];
    }
}

// ---- merge: the fold over a row's tile partials ------------------------------------------------
// The running maximum is a prefix maximum (exact under any association), so the coefficients of
// every step are computed in parallel and only `acc = fma(acc, a, part * b)` stays sequential.
constexpr int kMergeChunk = 1024;            // tiles folded per pass, at most (8 per thread)

// COLS = columns of the row per thread: the block has min(128, head_dim) threads (64 for
// head_dim <= 64), so no thread idles, and the fewer columns a thread carries the further ahead of
// its dependent chain it fetches the partials (256 / 8 / COLS ... tiles in flight).
template <int COLS>
__global__ void __launch_bounds__(kThreads)
merge_tiles_kernel(const AttnShape shape, const BatchMeta meta, const float* __restrict__ part_o,
                   const float* __restrict__ part_ml, int part_tiles, int world, int rank,
                   const EpilogueArgs ep) {
    __shared__ float coef_a[kMergeChunk];
    __shared__ float coef_b[kMergeChunk];
    __shared__ float part_l[kMergeChunk];
    __shared__ float warp_max[4];
    const int threads = blockDim.x;              // 64 or 128
    const int warps = threads >> 5;
    const int chunk_tiles = threads * 8;
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.x;
    const int b = blockIdx.y;
    const int d = shape.head_dim;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int position = meta.pos[b];
    int lo, first_tile, last_tile;
    tile_span(position, shape.window, lo, first_tile, last_tile);
    int n_tiles;
    if (world > 1) {
        const int first_owned = first_tile + ((rank - first_tile % world) + world) % world;
        n_tiles = first_owned > last_tile ? 0 : (last_tile - first_owned) / world + 1;
    } else {
        n_tiles = last_tile - first_tile + 1;
    }
    const size_t row = size_t(b) * shape.q_heads + head;

    float M, L;
    if (shape.count_sink) {
        const uint16_t bits = shape.sinks ? shape.sinks[head] : kNoSinkBits;
        M = __fmul_rn(bf16_bits_to_float(bits), kLog2e);
        L = 1.0f;
    } else {
        M = kEmptyMax;
        L = 0.0f;
    }
    constexpr int kCols = COLS;
    float A[kCols];
    #pragma unroll
    for (int cidx = 0; cidx < kCols; ++cidx) A[cidx] = 0.0f;

    for (int base = 0; base < n_tiles; base += chunk_tiles) {
        const int count = min(chunk_tiles, n_tiles - base);
        __syncthreads();
        // Thread t owns 8 consecutive tiles: local inclusive prefix maximum, then a block scan.
        float local[8];
        float running = __int_as_float(0xff800000);
        #pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int t = tid * 8 + u;
            const float mm = t < count ? part_ml[(row * part_tiles + base + t) * 2]
                                       : __int_as_float(0xff800000);
            local[u] = mm;
            running = fmaxf(running, mm);
        }
        float inclusive = running;
        #pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1) {
            const float other = __shfl_up_sync(0xffffffffu, inclusive, offset);
            if (lane >= offset) inclusive = fmaxf(inclusive, other);
        }
        if (lane == 31) warp_max[warp] = inclusive;
        __syncthreads();
        float before = M;                        // maximum of everything before this thread's tiles
        for (int w = 0; w < warp; ++w) before = fmaxf(before, warp_max[w]);
        const float prev_lane = __shfl_up_sync(0xffffffffu, inclusive, 1);
        if (lane > 0) before = fmaxf(before, prev_lane);
        #pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int t = tid * 8 + u;
            if (t < count) {
                float Mn, a, bcoef;
                fold_coefficients(before, local[u], Mn, a, bcoef);
                coef_a[t] = a;
                coef_b[t] = bcoef;
                part_l[t] = __fmul_rn(part_ml[(row * part_tiles + base + t) * 2 + 1], bcoef);
                before = Mn;
            }
        }
        float chunk_max = M;
        for (int w = 0; w < warps; ++w) chunk_max = fmaxf(chunk_max, warp_max[w]);
        __syncthreads();

        // The sequential part.  Every thread carries L (same chain, same bits) and its columns.
        const float* o_base = part_o + (row * part_tiles + base) * d;
        // The partials are fetched well ahead of the dependent chain that consumes them.
        constexpr int kAhead = 32 / COLS;
        for (int t0 = 0; t0 < count; t0 += kAhead) {
            float part[kAhead][kCols];
            #pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                #pragma unroll
                for (int cidx = 0; cidx < kCols; ++cidx) {
                    const int i = tid + cidx * threads;
                    part[u][cidx] = (t0 + u < count && i < d) ? __ldg(o_base + size_t(t0 + u) * d + i) : 0.0f;
                }
            }
            #pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                if (t0 + u < count) {
                    const float a = coef_a[t0 + u], bcoef = coef_b[t0 + u];
                    L = __fmaf_rn(L, a, part_l[t0 + u]);
                    #pragma unroll
                    for (int cidx = 0; cidx < kCols; ++cidx) {
                        A[cidx] = __fmaf_rn(A[cidx], a, __fmul_rn(part[u][cidx], bcoef));
                    }
                }
            }
        }
        M = chunk_max;
    }

    #pragma unroll
    for (int cidx = 0; cidx < kCols; ++cidx) {
        const int i = tid + cidx * threads;
        if (i < d) write_result(ep, size_t(b), shape.q_heads, head, d, i, A[cidx], M, L);
    }
}

// ---- prefill: one (kv head, token) per CTA, tiles folded in place ------------------------------
__global__ void __launch_bounds__(kThreads)
prefill_rows_kernel(const AttnShape shape, const CacheView cache, int seq,
                    const uint16_t* __restrict__ q, int first_position, const EpilogueArgs ep) {
    extern __shared__ __align__(16) unsigned char raw[];
    const int G = shape.group, d = shape.head_dim;
    const int kv_head = blockIdx.x;
    const int token = blockIdx.y;
    const int position = first_position + token;
    int lo, first_tile, last_tile;
    tile_span(position, shape.window, lo, first_tile, last_tile);

    float *A, *M, *L;
    SimtSmem sm = carve(raw, G, d, true, &A, &M, &L);
    load_group_queries(sm, q + (size_t(token) * shape.q_heads + size_t(kv_head) * G) * d, G, d);
    for (int i = threadIdx.x; i < G * d; i += kThreads) A[i] = 0.0f;
    if (threadIdx.x < G) {
        if (shape.count_sink) {
            const int head = kv_head * G + threadIdx.x;
            const uint16_t bits = shape.sinks ? shape.sinks[head] : kNoSinkBits;
            M[threadIdx.x] = __fmul_rn(bf16_bits_to_float(bits), kLog2e);
            L[threadIdx.x] = 1.0f;
        } else {
            M[threadIdx.x] = kEmptyMax;
            L[threadIdx.x] = 0.0f;
        }
    }
    __syncthreads();

    const size_t head_rows = (size_t(seq) * cache.kv_heads + kv_head) * cache.capacity;
    const int world = max(cache.map.world, 1);
    for (int tile = first_tile; tile <= last_tile; ++tile) {
        if (world > 1 && (tile % world) != cache.map.rank) continue;
        const size_t row0 = head_rows + row_of_tile(cache.map, tile);
        tile_partial(sm, cache.k + row0 * d, cache.v + row0 * d, tile * kTileKeys, lo, position, G,
                     d, shape.c);
        for (int i = threadIdx.x; i < G * d; i += kThreads) {
            const int g = i / d;
            float Mn, a, b;
            fold_coefficients(M[g], sm.mm[g], Mn, a, b);
            A[i] = fold_value(A[i], a, sm.acc[i], b);
        }
        __syncthreads();
        if (threadIdx.x < G) {
            const int g = threadIdx.x;
            float Mn, a, b;
            fold_coefficients(M[g], sm.mm[g], Mn, a, b);
            L[g] = __fmaf_rn(L[g], a, __fmul_rn(sm.l[g], b));
            M[g] = Mn;
        }
        __syncthreads();
    }

    for (int i = threadIdx.x; i < G * d; i += kThreads) {
        const int g = i / d;
        write_result(ep, size_t(token), shape.q_heads, kv_head * G + g, d, i - g * d, A[i], M[g], L[g]);
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
                       cudaStream_t stream) {
    if (tokens <= 0) return HC_OK;
    const size_t smem = simt_smem_bytes(shape.group, shape.head_dim, true);
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
            first_position + start, sub);
        ctx->launches += 1;
        err = cudaGetLastError();
        if (err != cudaSuccess) return check_cuda(err, "prefill_rows_kernel launch");
    }
    return HC_OK;
}

hc_status simt_decode(hc_context* ctx, const AttnShape& shape, const CacheView& cache,
                      const BatchMeta& meta, int n_seq, const uint16_t* q, const Workspace& ws,
                      const EpilogueArgs& ep, cudaStream_t stream) {
    if (n_seq <= 0) return HC_OK;
    const int world = cache.map.world > 1 ? cache.map.world : 1;
    int max_tiles = 0;
    for (int b = 0; b < n_seq; ++b) {
        int lo, first_tile, last_tile;
        tile_span(meta.pos[b], shape.window, lo, first_tile, last_tile);
        int n = last_tile - first_tile + 1;
        if (world > 1) n = (n + world - 1) / world + 1;
        if (n > max_tiles) max_tiles = n;
    }
    const size_t rows = size_t(n_seq) * shape.q_heads;
    if (rows * max_tiles * shape.head_dim > ws.part_o_floats || rows * max_tiles * 2 > ws.part_ml_floats) {
        return fail(HC_KV_OVERFLOW, "decode: the split-attention workspace is too small for this call");
    }
    const size_t smem = simt_smem_bytes(shape.group, shape.head_dim, false);
    cudaError_t err = cudaFuncSetAttribute(decode_tiles_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (err != cudaSuccess) return check_cuda(err, "decode_tiles_kernel shared memory");
    dim3 grid(max_tiles, shape.kv_heads, n_seq);
    decode_tiles_kernel<<<grid, kThreads, smem, stream>>>(shape, cache, meta, q, ws.part_o,
                                                         ws.part_ml, max_tiles);
    ctx->launches += 1;
    err = cudaGetLastError();
    if (err != cudaSuccess) return check_cuda(err, "decode_tiles_kernel launch");
    return launch_merge(ctx, shape, meta, n_seq, ws, max_tiles, world, cache.map.rank, ep, stream);
}

hc_status launch_merge(hc_context* ctx, const AttnShape& shape, const BatchMeta& meta, int n_seq,
                       const Workspace& ws, int part_tiles, int world, int rank, const EpilogueArgs& ep,
                       cudaStream_t stream) {
    dim3 mgrid(shape.q_heads, n_seq);
    const int d = shape.head_dim;
    const int threads = d <= 64 ? 64 : kThreads;
    const int cols = (d + threads - 1) / threads;
    auto kernel = cols <= 1 ? merge_tiles_kernel<1> : cols == 2 ? merge_tiles_kernel<2> : merge_tiles_kernel<4>;
    const cudaError_t launched = launch_pdl(kernel, mgrid, dim3(threads), 0, stream, shape, meta,
                                            static_cast<const float*>(ws.part_o), static_cast<const float*>(ws.part_ml),
                                            part_tiles, world, rank, ep);
    ctx->launches += 1;
    if (launched != cudaSuccess) return check_cuda(launched, "merge_tiles_kernel launch");
    return check_cuda(cudaGetLastError(), "merge_tiles_kernel launch");
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
    int max_tiles = 0;
    for (int b = 0; b < n_seq; ++b) {
        int lo, first_tile, last_tile;
        tile_span(meta.pos[b], shape.window, lo, first_tile, last_tile);
        max_tiles = std::max(max_tiles, last_tile - first_tile + 1);
    }
    // Partials: [rows][tiles][d] then [rows][tiles][2].
    const size_t rows = size_t(n_seq) * shape.q_heads;
    const size_t o_floats = rows * max_tiles * shape.head_dim;
    const size_t need = o_floats + rows * max_tiles * 2;
    if (need > kStaticScratchFloats) {
        return fail(HC_KV_OVERFLOW, "hc_attention_decode_static: this call needs " + std::to_string(need * 4) +
                                        " bytes of partials, the fixed scratch holds " +
                                        std::to_string(kStaticScratchFloats * 4));
    }
    // Every partial the merge reads is written by this call's split kernel first, so nothing in the
    // array has to start at zero.
    Workspace ws;
    ws.part_o = ctx->static_scratch;
    ws.part_ml = ctx->static_scratch + o_floats;
    ws.part_o_floats = o_floats;
    ws.part_ml_floats = rows * max_tiles * 2;
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
