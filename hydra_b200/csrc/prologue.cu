// prologue.cu — everything that happens to q, k and v before attention, in one kernel:
// per-head RMSNorm, half-split rotation, rounding to bf16 and, for k and v, the store into the
// cache.  Also the stand-alone element-wise kernels of the protocol.
//
// Replaces, fused: rms_norm_heads (Sources/HydraMetal/Shaders/gemma.metal:785-821), rope_apply /
// rope_apply_batch / rope_apply_batched (attention.metal:48-72, batch.metal:224-251,
// gemma.metal:961-984) and kv_cache_write / kv_cache_write_batch (dense.metal:66-86,
// batch.metal:254-277).  The order is the reference's: norm, then rotation, then the cast
// (Sources/HydraReference/Gemma4ReferenceLayer.swift:154-157, 234-246); v is normalised without a
// weight and never rotated.
//
// HBM-bound and tiny: a chunk of 512 tokens moves a few MB, so what matters is how many bytes each
// warp has in flight.

#include <algorithm>

#include "internal.hpp"

namespace hc {
namespace {

constexpr int kPrepWarps = 8;
constexpr int kMaxHeadDim = 512;

// Four consecutive elements of an activation row as fp32 (8-byte load for bf16, 16-byte for fp32).
__device__ __forceinline__ void load_io4(const void* base, size_t index, int dtype, float (&out)[4]) {
    if (dtype == 0) {
        const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + index);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    } else {
        const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(base) + index);
        out[0] = bf16_bits_to_float(uint16_t(v.x & 0xffffu));
        out[1] = bf16_bits_to_float(uint16_t(v.x >> 16));
        out[2] = bf16_bits_to_float(uint16_t(v.y & 0xffffu));
        out[3] = bf16_bits_to_float(uint16_t(v.y >> 16));
    }
}
__device__ __forceinline__ uint2 pack_bf16x4(const float (&v)[4]) {
    uint2 r;
    r.x = uint32_t(float_to_bf16_bits(v[0])) | (uint32_t(float_to_bf16_bits(v[1])) << 16);
    r.y = uint32_t(float_to_bf16_bits(v[2])) | (uint32_t(float_to_bf16_bits(v[3])) << 16);
    return r;
}
__device__ __forceinline__ void store_io4(void* base, size_t index, int dtype, const float (&v)[4]) {
    if (dtype == 0) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + index) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(base) + index) = pack_bf16x4(v);
    }
}

// The kernel for head_dim 64, 128 and 256 (LPV = head_dim / 8 lanes per head vector, so a warp holds
// 4, 2 or 1 vectors at a time).  Lane m of a vector owns elements 4m..4m+3 of each half, which keeps
// both members of every rotation pair (i, i + d/2) in one lane and makes every access an 8- or 16-byte
// one.  The launcher checks the alignment this needs and otherwise uses the general kernel below.
template <int LPV>
__global__ void __launch_bounds__(kPrepWarps * 32)
prepare_heads_vec_kernel(const PrepArgs args, int total_heads) {
    constexpr int d = 8 * LPV;
    constexpr int half = 4 * LPV;
    constexpr int kPerWarp = 32 / LPV;
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int sub = lane / LPV;
    const int m = lane % LPV;
    // 32-bit indices: a launch covers at most 32768 tokens x a few hundred heads.
    const unsigned vectors = unsigned(args.tokens) * unsigned(total_heads);
    const unsigned groups = (vectors + kPerWarp - 1) / kPerWarp;
    const unsigned stride = gridDim.x * kPrepWarps;
    for (unsigned grp = blockIdx.x * kPrepWarps + warp; grp < groups; grp += stride) {
        unsigned vec = grp * kPerWarp + sub;
        bool active = vec < vectors;
        if (!active) vec = vectors - 1;              // keeps the lane's loads legal; nothing is stored
        const int token = int(vec / unsigned(total_heads));
        int head = int(vec - unsigned(token) * unsigned(total_heads));
        int job_index = 0;
        while (head >= args.job[job_index].heads) {
            head -= args.job[job_index].heads;
            ++job_index;
        }
        const PrepJob& job = args.job[job_index];
        const int position = args.batched ? args.meta.pos[token] : args.first_position + token;
        const int seq = args.batched ? args.meta.seq[token] : args.seq;
        const bool to_cache = job.kind == 1 || job.kind == 2;
        if (to_cache && !row_is_local(args.cache.map, position)) active = false;   // another rank's tile

        const size_t src_base = size_t(token) * size_t(job.token_stride) + size_t(head) * job.head_stride;
        float x[8];
        {
            float lo[4], hi[4];
            load_io4(job.src, src_base + 4 * m, job.src_dtype, lo);
            load_io4(job.src, src_base + half + 4 * m, job.src_dtype, hi);
            #pragma unroll
            for (int j = 0; j < 4; ++j) { x[j] = lo[j]; x[4 + j] = hi[j]; }
        }
        float4 cosv = make_float4(1.0f, 1.0f, 1.0f, 1.0f), sinv = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (job.rope != 0) {
            const int table_row = position < args.table_positions ? position : args.table_positions - 1;
            cosv = *reinterpret_cast<const float4*>(args.cos + size_t(table_row) * half + 4 * m);
            sinv = *reinterpret_cast<const float4*>(args.sin + size_t(table_row) * half + 4 * m);
        }
        if (job.norm != 0) {
            float sum = 0.0f;
            #pragma unroll
            for (int j = 0; j < 8; ++j) sum = __fmaf_rn(x[j], x[j], sum);
            #pragma unroll
            for (int offset = LPV / 2; offset > 0; offset >>= 1) {
                sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, offset));
            }
            const float inverse = __frsqrt_rn(__fadd_rn(__fdiv_rn(sum, float(d)), args.eps));
            #pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = __fmul_rn(x[j], inverse);
            if (job.norm == 1) {
                float wl[4], wh[4];
                load_io4(job.weight, size_t(4 * m), 1, wl);
                load_io4(job.weight, size_t(half + 4 * m), 1, wh);
                #pragma unroll
                for (int j = 0; j < 4; ++j) {
                    x[j] = __fmul_rn(x[j], wl[j]);
                    x[4 + j] = __fmul_rn(x[4 + j], wh[j]);
                }
            }
        }
        float lo[4], hi[4];
        if (job.rope != 0) {
            const float c[4] = {cosv.x, cosv.y, cosv.z, cosv.w};
            const float s[4] = {sinv.x, sinv.y, sinv.z, sinv.w};
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                lo[j] = __fmaf_rn(x[j], c[j], -__fmul_rn(x[4 + j], s[j]));
                hi[j] = __fmaf_rn(x[4 + j], c[j], __fmul_rn(x[j], s[j]));
            }
        } else {
            #pragma unroll
            for (int j = 0; j < 4; ++j) { lo[j] = x[j]; hi[j] = x[4 + j]; }
        }
        if (!active) continue;
        if (job.kind == 3) {
            store_io4(job.dst, src_base + 4 * m, job.src_dtype, lo);
            store_io4(job.dst, src_base + half + 4 * m, job.src_dtype, hi);
        } else {
            uint16_t* dst16;
            if (job.kind == 0) {
                dst16 = reinterpret_cast<uint16_t*>(job.dst) + (size_t(token) * job.heads + head) * d;
            } else {
                const int row = cache_row(args.cache.map, seq, position);
                uint16_t* base = job.kind == 1 ? args.cache.k : args.cache.v;
                dst16 = base + (size_t(cache_plane(args.cache.map, seq, args.cache.kv_heads, head)) * args.cache.capacity + row) * d;
            }
            *reinterpret_cast<uint2*>(dst16 + 4 * m) = pack_bf16x4(lo);
            *reinterpret_cast<uint2*>(dst16 + half + 4 * m) = pack_bf16x4(hi);
        }
    }
}

// The general kernel: any even head_dim up to 512, any alignment.  One warp per head vector, staged
// in shared memory.
__global__ void __launch_bounds__(kPrepWarps * 32)
prepare_heads_kernel(const PrepArgs args) {
    __shared__ float stage[kPrepWarps][kMaxHeadDim];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int d = args.head_dim;
    const int half = d >> 1;

    int total_heads = 0;
    for (int j = 0; j < args.n_jobs; ++j) total_heads += args.job[j].heads;
    // Warps stride over the (token, head) vectors of the call.
    // 32-bit indices: a launch covers at most 32768 tokens x a few hundred heads.
    const unsigned vectors = unsigned(args.tokens) * unsigned(total_heads);
    const unsigned stride = gridDim.x * kPrepWarps;
    for (unsigned vec = blockIdx.x * kPrepWarps + warp; vec < vectors; vec += stride) {
    const int token = int(vec / unsigned(total_heads));
    const int slot = int(vec - unsigned(token) * unsigned(total_heads));
    int job_index = 0, head = slot;
    while (head >= args.job[job_index].heads) {
        head -= args.job[job_index].heads;
        ++job_index;
    }
    const PrepJob& job = args.job[job_index];

    const int position = args.batched ? args.meta.pos[token] : args.first_position + token;
    const int seq = args.batched ? args.meta.seq[token] : args.seq;
    if (job.kind == 1 || job.kind == 2) {
        if (!row_is_local(args.cache.map, position)) continue;   // another rank owns this key tile
    }

    const size_t src_base = size_t(token) * size_t(job.token_stride) + size_t(head) * job.head_stride;
    const bool rotate = job.rope != 0;
    const int table_row = position < args.table_positions ? position : args.table_positions - 1;
    // Destination of this head vector.
    uint16_t* dst16 = nullptr;
    if (job.kind == 0) {
        dst16 = reinterpret_cast<uint16_t*>(job.dst) + (size_t(token) * job.heads + head) * d;
    } else if (job.kind == 1 || job.kind == 2) {
        const int row = cache_row(args.cache.map, seq, position);
        uint16_t* base = job.kind == 1 ? args.cache.k : args.cache.v;
        dst16 = base + (size_t(cache_plane(args.cache.map, seq, args.cache.kv_heads, head)) * args.cache.capacity + row) * d;
    }

    // Stage the vector in shared memory.
    __syncwarp();                                  // the staging row is reused
    float* x = stage[warp];
    float sum = 0.0f;
    for (int i = lane; i < d; i += 32) {
        const float value = load_io(job.src, src_base + i, job.src_dtype);
        x[i] = value;
        sum = __fmaf_rn(value, value, sum);
    }
    if (job.norm != 0) {
        #pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, offset));
        }
        const float inverse = __frsqrt_rn(__fadd_rn(__fdiv_rn(sum, float(d)), args.eps));
        for (int i = lane; i < d; i += 32) {
            float value = __fmul_rn(x[i], inverse);
            if (job.norm == 1) value = __fmul_rn(value, bf16_bits_to_float(job.weight[i]));
            x[i] = value;
        }
    }
    __syncwarp();
    for (int i = lane; i < half; i += 32) {
        float x1 = x[i], x2 = x[half + i];
        if (rotate) {
            const float c = args.cos[size_t(table_row) * half + i];
            const float s = args.sin[size_t(table_row) * half + i];
            const float r1 = __fmaf_rn(x1, c, -__fmul_rn(x2, s));
            const float r2 = __fmaf_rn(x2, c, __fmul_rn(x1, s));
            x1 = r1;
            x2 = r2;
        }
        if (job.kind == 3) {
            store_io(job.dst, src_base + i, job.src_dtype, x1);
            store_io(job.dst, src_base + half + i, job.src_dtype, x2);
        } else {
            dst16[i] = float_to_bf16_bits(x1);
            dst16[half + i] = float_to_bf16_bits(x2);
        }
    }
    }
}

// RMSNorm of whole rows (the layer's input norm): out = x * rsqrt(mean(x^2) + eps) * scale.  One block
// per token; replaces rms_norm and rms_norm_batch (Sources/HydraMetal/Shaders/attention.metal:9-43,
// batch.metal:184-218).  The output may be bf16, ready to be the A operand of hc_linear.
// Rows whose width is a multiple of 4 (and at most 4096) are read once, four elements per load, and
// kept in registers between the sum and the scaling: all of a thread's loads are in flight together,
// where an element-by-element loop with the dtype looked up per element paid one memory round trip
// after the other (12 us for one 2880-wide row).  The sum's order is fixed by the width alone.
constexpr int kNormVecs = 4;      // float4 per thread held in registers: 256 threads x 16 values

__device__ __forceinline__ float4 load_io4(const void* p, size_t index, int dtype) {
    if (dtype == HC_F32) return *reinterpret_cast<const float4*>(static_cast<const float*>(p) + index);
    const uint2 bits = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p) + index);
    return make_float4(__uint_as_float(bits.x << 16), __uint_as_float(bits.x & 0xffff0000u),
                       __uint_as_float(bits.y << 16), __uint_as_float(bits.y & 0xffff0000u));
}

__global__ void __launch_bounds__(256)
rms_norm_rows_kernel(const void* __restrict__ x, const uint16_t* __restrict__ scale, void* __restrict__ out, int width,
                     float eps, int x_dtype, int out_dtype, int vectors) {
    __shared__ float warp_sum[8];
    __shared__ float inverse;
    const size_t base = size_t(blockIdx.x) * width;
    float partial = 0.0f;
    float4 held[kNormVecs];
    if (vectors) {
        #pragma unroll
        for (int u = 0; u < kNormVecs; ++u) {
            const int i = (threadIdx.x + u * 256) * 4;
            held[u] = i < width ? load_io4(x, base + i, x_dtype) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        #pragma unroll
        for (int u = 0; u < kNormVecs; ++u) {
            partial = __fmaf_rn(held[u].x, held[u].x, partial);
            partial = __fmaf_rn(held[u].y, held[u].y, partial);
            partial = __fmaf_rn(held[u].z, held[u].z, partial);
            partial = __fmaf_rn(held[u].w, held[u].w, partial);
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float v = load_io(x, base + i, x_dtype);
            partial = __fmaf_rn(v, v, partial);
        }
    }
    #pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, offset);
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = partial;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int w = 0; w < int(blockDim.x >> 5); ++w) total += warp_sum[w];
        inverse = rsqrtf(total / float(width) + eps);
    }
    __syncthreads();
    const float inv = inverse;
    if (vectors) {
        #pragma unroll
        for (int u = 0; u < kNormVecs; ++u) {
            const int i = (threadIdx.x + u * 256) * 4;
            if (i >= width) continue;
            float w[4] = {1.0f, 1.0f, 1.0f, 1.0f};
            if (scale != nullptr) {
                const uint2 bits = *reinterpret_cast<const uint2*>(scale + i);
                w[0] = __uint_as_float(bits.x << 16);
                w[1] = __uint_as_float(bits.x & 0xffff0000u);
                w[2] = __uint_as_float(bits.y << 16);
                w[3] = __uint_as_float(bits.y & 0xffff0000u);
            }
            const float r0 = __fmul_rn(__fmul_rn(held[u].x, inv), w[0]), r1 = __fmul_rn(__fmul_rn(held[u].y, inv), w[1]);
            const float r2 = __fmul_rn(__fmul_rn(held[u].z, inv), w[2]), r3 = __fmul_rn(__fmul_rn(held[u].w, inv), w[3]);
            if (out_dtype == HC_F32) {
                *reinterpret_cast<float4*>(static_cast<float*>(out) + base + i) = make_float4(r0, r1, r2, r3);
            } else {
                uint2 packed;
                packed.x = uint32_t(float_to_bf16_bits(r0)) | (uint32_t(float_to_bf16_bits(r1)) << 16);
                packed.y = uint32_t(float_to_bf16_bits(r2)) | (uint32_t(float_to_bf16_bits(r3)) << 16);
                *reinterpret_cast<uint2*>(static_cast<uint16_t*>(out) + base + i) = packed;
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = load_io(x, base + i, x_dtype);
        const float w = scale != nullptr ? bf16_bits_to_float(scale[i]) : 1.0f;
        store_io(out, base + i, out_dtype, __fmul_rn(__fmul_rn(v, inv), w));
    }
}

__global__ void split_query_gate_kernel(const void* combined, void* query, void* gate, size_t count,
                                        int d, int dtype) {
    // count = tokens * heads * d; element e = (token*heads + head) * d + i
    const size_t e = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= count) return;
    const size_t vec = e / d;
    const int i = int(e % d);
    store_io(query, e, dtype, load_io(combined, vec * 2 * d + i, dtype));
    store_io(gate, e, dtype, load_io(combined, vec * 2 * d + d + i, dtype));
}

__global__ void output_gate_kernel(void* output, const void* gate, size_t count, int dtype) {
    const size_t e = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= count) return;
    const float value = load_io(output, e, dtype);
    store_io(output, e, dtype, __fmul_rn(value, sigmoid_gate(load_io(gate, e, dtype))));
}

}  // namespace

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

hc_status launch_prepare(hc_context* ctx, const PrepArgs& args, cudaStream_t stream) {
    int total_heads = 0;
    for (int j = 0; j < args.n_jobs; ++j) total_heads += args.job[j].heads;
    if (total_heads == 0 || args.tokens == 0) return HC_OK;
    const long long vectors = (long long)args.tokens * total_heads;
    const int d = args.head_dim;
    const long long cap = (long long)std::max(ctx->sm_count, 1) * 16;
    // The vector kernel needs 16-byte aligned rows everywhere it touches.
    bool vector_ok = d == 64 || d == 128 || d == 256;
    for (int j = 0; j < args.n_jobs && vector_ok; ++j) {
        const PrepJob& job = args.job[j];
        if (job.heads == 0) continue;
        vector_ok = aligned16(job.src) && job.token_stride % 8 == 0 && job.head_stride % 8 == 0 &&
                    (job.norm != 1 || aligned16(job.weight)) &&
                    ((job.kind != 0 && job.kind != 3) || aligned16(job.dst));
    }
    if (vector_ok) {
        const int per_warp = 256 / d;
        const long long groups = (vectors + per_warp - 1) / per_warp;
        const int grid = int(std::min<long long>((groups + kPrepWarps - 1) / kPrepWarps, cap));
        if (d == 64) launch_pdl(prepare_heads_vec_kernel<8>, grid, kPrepWarps * 32, 0, stream, args, total_heads);
        else if (d == 128) launch_pdl(prepare_heads_vec_kernel<16>, grid, kPrepWarps * 32, 0, stream, args, total_heads);
        else launch_pdl(prepare_heads_vec_kernel<32>, grid, kPrepWarps * 32, 0, stream, args, total_heads);
    } else {
        const long long wanted = (vectors + kPrepWarps - 1) / kPrepWarps;
        const int grid = int(std::min<long long>(wanted, cap));
        launch_pdl(prepare_heads_kernel, grid, kPrepWarps * 32, 0, stream, args);
    }
    ctx->launches += 1;
    return check_cuda(cudaGetLastError(), "prepare_heads_kernel launch");
}

hc_status launch_rms_norm_rows(hc_context* ctx, const void* x, const uint16_t* scale, void* out, int tokens, int width,
                               float eps, int x_dtype, int out_dtype, cudaStream_t stream) {
    if (tokens <= 0) return HC_OK;
    // Four elements per load where every row starts on a 16-byte boundary in every buffer it touches.
    const bool vectors = width % 4 == 0 && width <= 256 * 4 * 4 && aligned16(x) && aligned16(out) &&
                         (scale == nullptr || (reinterpret_cast<uintptr_t>(scale) & 7u) == 0) &&
                         (width % 8 == 0 || (x_dtype == HC_F32 && out_dtype == HC_F32));
    rms_norm_rows_kernel<<<unsigned(tokens), 256, 0, stream>>>(x, scale, out, width, eps, x_dtype, out_dtype, vectors ? 1 : 0);
    ctx->launches += 1;
    return check_cuda(cudaGetLastError(), "rms_norm_rows_kernel launch");
}

hc_status launch_split_query_gate(hc_context* ctx, const void* combined, void* query, void* gate,
                                  int tokens, int heads, int d, int dtype, cudaStream_t stream) {
    const size_t count = size_t(tokens) * heads * d;
    if (count == 0) return HC_OK;
    split_query_gate_kernel<<<unsigned((count + 255) / 256), 256, 0, stream>>>(combined, query, gate,
                                                                               count, d, dtype);
    ctx->launches += 1;
    return check_cuda(cudaGetLastError(), "split_query_gate_kernel launch");
}

hc_status launch_output_gate(hc_context* ctx, void* output, const void* gate, size_t count,
                             int dtype, cudaStream_t stream) {
    if (count == 0) return HC_OK;
    output_gate_kernel<<<unsigned((count + 255) / 256), 256, 0, stream>>>(output, gate, count, dtype);
    ctx->launches += 1;
    return check_cuda(cudaGetLastError(), "output_gate_kernel launch");
}

}  // namespace hc
