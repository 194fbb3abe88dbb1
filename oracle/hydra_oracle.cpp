// hydra_oracle.cpp — CPU restatement of Hydra's double-precision attention reference.
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are compared with and the
// CPU baseline that the benchmark times.  Nothing in the product library links, loads or calls it.
//
// The reference oracle (`Sources/HydraReference`, Swift) cannot be built where this runs: there is
// no Swift toolchain.  Every function below restates one reference function in double precision
// with the same loop structure (two-pass softmax: maximum, then sum; explicit dot products) and
// cites the file:line it follows.  The restatement is pinned by the reference's own golden vectors
// (`Tests/HydraReferenceTests/Fixtures/reference_ops.json`, `gemma4_operators.json`) and by vectors
// produced by the reference's pure-Python transcriptions (`tools/gen_reference_fixtures.py`,
// `tools/gen_gemma_fixtures.py`); see tests/golden/.
//
// Build: g++ -O2 -std=c++17 -shared -fPIC -pthread hydra_oracle.cpp -o libhydra_oracle.so
//
// All entry points are extern "C" over plain pointers so that Python (ctypes) can call them.

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace {

// ---- bf16 -------------------------------------------------------------------------------------
// Sources/HydraFormat/BF16.swift:20-32 — round to nearest, ties to even; NaN keeps its top bits
// and gets the quiet bit.
inline uint16_t bf16_from_float(float value) {
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    if (std::isnan(value)) return static_cast<uint16_t>((bits >> 16) | 0x0040u);
    const uint32_t rounding = 0x7FFFu + ((bits >> 16) & 1u);
    return static_cast<uint16_t>((bits + rounding) >> 16);
}
inline float bf16_to_float(uint16_t bits) {
    const uint32_t wide = static_cast<uint32_t>(bits) << 16;
    float out;
    std::memcpy(&out, &wide, 4);
    return out;
}

// ---- RMSNorm ----------------------------------------------------------------------------------
// Sources/HydraReference/Gemma4ReferenceOps.swift:25-31 — x * (mean(x^2) + eps)^-0.5 * w, the
// weight is w (not 1 + w); weight == nullptr is the weightless form (Gemma's v_norm).
// Sources/HydraReference/ReferenceOps.swift:20-25 is the same function written with
// 1 / sqrt(mean + eps); `use_sqrt` selects that spelling so both fixtures reproduce to the last bit
// they can.
template <typename T>
void rms_norm(const T* x, const double* weight, int n, double eps, bool use_sqrt, double* out) {
    double sum = 0.0;
    for (int i = 0; i < n; ++i) sum += double(x[i]) * double(x[i]);
    const double mean = sum / double(n);
    const double scale = use_sqrt ? 1.0 / std::sqrt(mean + eps) : std::pow(mean + eps, -0.5);
    for (int i = 0; i < n; ++i) {
        out[i] = weight ? double(x[i]) * scale * weight[i] : double(x[i]) * scale;
    }
}

// ---- RoPE -------------------------------------------------------------------------------------
// Sources/HydraReference/ReferenceOps.swift:65-75 and Gemma4ReferenceOps.swift:70-82 — split into
// two halves: pair (i, i + d/2).
void apply_rope(const double* x, int d, const double* cosv, const double* sinv, double* out) {
    const int half = d / 2;
    for (int i = 0; i < half; ++i) {
        const double x1 = x[i], x2 = x[half + i];
        out[i] = x1 * cosv[i] - x2 * sinv[i];
        out[half + i] = x2 * cosv[i] + x1 * sinv[i];
    }
}

// One query row against a key range.  This is the loop body of ReferenceOps.sdpa
// (Sources/HydraReference/ReferenceOps.swift:128-158) and of ReferenceLayer.decode
// (Sources/HydraReference/ReferenceLayer.swift:152-183): logits = dot * scale, peak starts at the
// sink, denominator = exp(sink - peak) + sum exp(logit - peak), out += weight * v.  `has_sink == 0`
// is Gemma4ReferenceOps.attention + softmax (Gemma4ReferenceOps.swift:93-118): peak = max logit and
// nothing is added to the denominator.
//
// K and V are addressed as base + key * stride (elements), so the same routine serves the
// reference's [position][kvHeads*headDim] history and a per-head contiguous history.
template <typename T>
void attend_row(const double* q, const T* k, const T* v, ptrdiff_t stride, int first, int last,
                int d, double scale, int has_sink, double sink, double* out,
                std::vector<double>& logits) {
    const int count = last - first + 1;
    logits.resize(size_t(count));
    double peak = has_sink ? sink : -std::numeric_limits<double>::infinity();
    for (int key = first; key <= last; ++key) {
        const T* row = k + ptrdiff_t(key) * stride;
        double dot = 0.0;
        for (int i = 0; i < d; ++i) dot += q[i] * double(row[i]);
        const double logit = dot * scale;
        logits[size_t(key - first)] = logit;
        peak = std::max(peak, logit);
    }
    double denominator = has_sink ? std::exp(sink - peak) : 0.0;
    for (int j = 0; j < count; ++j) denominator += std::exp(logits[size_t(j)] - peak);
    for (int i = 0; i < d; ++i) out[i] = 0.0;
    for (int key = first; key <= last; ++key) {
        const double weight = std::exp(logits[size_t(key - first)] - peak) / denominator;
        const T* row = v + ptrdiff_t(key) * stride;
        for (int i = 0; i < d; ++i) out[i] += weight * double(row[i]);
    }
}

template <typename F>
void parallel_for(int n, int threads, F&& body) {
    if (threads <= 1 || n <= 1) {
        for (int i = 0; i < n; ++i) body(i);
        return;
    }
    std::atomic<int> next{0};
    std::vector<std::thread> pool;
    const int count = std::min(threads, n);
    pool.reserve(size_t(count));
    for (int t = 0; t < count; ++t) {
        pool.emplace_back([&]() {
            for (;;) {
                const int i = next.fetch_add(1);
                if (i >= n) break;
                body(i);
            }
        });
    }
    for (auto& th : pool) th.join();
}

inline double sigmoid(double x) { return 1.0 / (1.0 + std::exp(-x)); }

}  // namespace

extern "C" {

int ho_hardware_threads() {
    const unsigned n = std::thread::hardware_concurrency();
    return n == 0 ? 1 : int(n);
}

// ---- bf16 helpers (Sources/HydraFormat/BF16.swift:20-32) --------------------------------------
void ho_bf16_round(const float* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = bf16_to_float(bf16_from_float(in[i]));
}
void ho_bf16_encode(const float* in, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = bf16_from_float(in[i]);
}
void ho_bf16_decode(const uint16_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = bf16_to_float(in[i]);
}

// ---- RMSNorm ----------------------------------------------------------------------------------
void ho_rms_norm(const double* x, const double* weight, int n, double eps, int use_sqrt,
                 double* out) {
    rms_norm(x, weight, n, eps, use_sqrt != 0, out);
}

// ---- RoPE tables ------------------------------------------------------------------------------
// Sources/HydraCore/RoPETables.swift:54-85 — inverse frequencies with the YaRN extension.
// scaling_factor <= 1 is plain RoPE: 1 / base^(2i/d), concentration 1.
// Returns 0, or -1 if the YaRN bounds are inconsistent (the reference traps on that).
int ho_yarn_inverse_frequencies(int head_dim, double base, int initial_context, double scaling,
                                double ntk_alpha, double ntk_beta, double* inv_freq,
                                double* concentration) {
    const int pairs = head_dim / 2;
    std::vector<double> freq(size_t(pairs), 0.0);
    for (int i = 0; i < pairs; ++i) freq[size_t(i)] = std::pow(base, double(2 * i) / double(head_dim));
    if (!(scaling > 1.0)) {
        *concentration = 1.0;
        for (int i = 0; i < pairs; ++i) inv_freq[i] = 1.0 / freq[size_t(i)];
        return 0;
    }
    *concentration = 0.1 * std::log(scaling) + 1.0;
    const double half_dim = double(head_dim) / 2.0;
    const double context = double(initial_context);
    const double pi = 3.14159265358979323846;
    const double low = half_dim * std::log(context / (ntk_beta * 2 * pi)) / std::log(base);
    const double high = half_dim * std::log(context / (ntk_alpha * 2 * pi)) / std::log(base);
    if (!(low > 0 && low < high && high < half_dim - 1)) return -1;
    for (int i = 0; i < pairs; ++i) {
        const double interpolation = 1.0 / (scaling * freq[size_t(i)]);
        const double extrapolation = 1.0 / freq[size_t(i)];
        const double ramp = (double(i) - low) / (high - low);
        const double mask = 1.0 - std::min(std::max(ramp, 0.0), 1.0);
        inv_freq[i] = interpolation * (1.0 - mask) + extrapolation * mask;
    }
    return 0;
}

// Sources/HydraReference/Gemma4ReferenceOps.swift:55-64 and RoPETables.swift:127-143 — plain
// frequencies theta^(-2i/d) for the first `rotating_pairs` pairs, zero for the rest (partial rotary).
void ho_inverse_frequencies(int head_dim, double theta, int rotating_pairs, double* inv_freq) {
    const int pairs = head_dim / 2;
    for (int i = 0; i < pairs; ++i) inv_freq[i] = 0.0;
    for (int i = 0; i < std::min(std::max(rotating_pairs, 0), pairs); ++i) {
        inv_freq[i] = 1.0 / std::pow(theta, 2.0 * double(i) / double(head_dim));
    }
}

// Sources/HydraCore/RoPETables.swift:89-95 — cos(t * f) * concentration, sin(t * f) * concentration.
void ho_rope_tables(const double* inv_freq, int pairs, double concentration, const int64_t* positions,
                    int n_positions, double* cos_out, double* sin_out) {
    for (int p = 0; p < n_positions; ++p) {
        const double t = double(positions[p]);
        for (int i = 0; i < pairs; ++i) {
            cos_out[size_t(p) * pairs + i] = std::cos(t * inv_freq[i]) * concentration;
            sin_out[size_t(p) * pairs + i] = std::sin(t * inv_freq[i]) * concentration;
        }
    }
}

// Sources/HydraCore/RoPETables.swift:98-107 — the run-time tables: the same values cast to Float.
void ho_rope_tables_f32(const double* inv_freq, int pairs, double concentration,
                        const int64_t* positions, int n_positions, float* cos_out, float* sin_out) {
    for (int p = 0; p < n_positions; ++p) {
        const double t = double(positions[p]);
        for (int i = 0; i < pairs; ++i) {
            cos_out[size_t(p) * pairs + i] = float(std::cos(t * inv_freq[i]) * concentration);
            sin_out[size_t(p) * pairs + i] = float(std::sin(t * inv_freq[i]) * concentration);
        }
    }
}

// Sources/HydraReference/ReferenceOps.swift:65-75 — one head vector, tables given.
void ho_apply_rope(const double* x, int head_dim, const double* cosv, const double* sinv,
                   double* out) {
    apply_rope(x, head_dim, cosv, sinv, out);
}

// Sources/HydraReference/Gemma4ReferenceOps.swift:70-82 — one head vector, angle = position * f.
void ho_apply_rope_position(const double* x, int head_dim, int64_t position, const double* inv_freq,
                            double* out) {
    const int half = head_dim / 2;
    std::vector<double> c(size_t(half), 0.0), s(size_t(half), 0.0);
    for (int i = 0; i < half; ++i) {
        const double angle = double(position) * inv_freq[i];
        c[size_t(i)] = std::cos(angle);
        s[size_t(i)] = std::sin(angle);
    }
    apply_rope(x, head_dim, c.data(), s.data(), out);
}

// ---- Attention --------------------------------------------------------------------------------
// Sources/HydraReference/ReferenceOps.swift:116-163 — sdpa with sinks and an optional window.
// q [tokens][kvHeads][qMult][d]; k, v [tokens][kvHeads][d]; sinks [kvHeads*qMult];
// out [tokens][kvHeads*qMult*d].  Key `key` is skipped when key <= query - window.
void ho_sdpa(const double* q, const double* k, const double* v, const double* sinks, int tokens,
             int kv_heads, int q_mult, int d, double sm_scale, int window, double* out) {
    std::vector<double> logits;
    for (int h = 0; h < kv_heads; ++h) {
        for (int m = 0; m < q_mult; ++m) {
            const double sink = sinks[h * q_mult + m];
            for (int query = 0; query < tokens; ++query) {
                const int first = window > 0 ? std::max(0, query - window + 1) : 0;
                const double* qrow = q + ((size_t(query) * kv_heads + h) * q_mult + m) * d;
                attend_row(qrow, k + size_t(h) * d, v + size_t(h) * d, ptrdiff_t(kv_heads) * d,
                           first, query, d, sm_scale, 1, sink,
                           out + size_t(query) * kv_heads * q_mult * d + size_t(h * q_mult + m) * d,
                           logits);
            }
        }
    }
}

// Sources/HydraReference/Gemma4ReferenceOps.swift:93-118 — one query against a history, scale 1.0,
// no sink, window = the last `window` keys.
void ho_gemma_attention(const double* query, const double* keys, const double* values, int n_keys,
                        int d, int window, double* out) {
    std::vector<double> logits;
    const int first = window == 0 ? 0 : std::max(0, n_keys - window);
    attend_row(query, keys, values, ptrdiff_t(d), first, n_keys - 1, d, 1.0, 0, 0.0, out, logits);
}

// Sources/HydraReference/QwenReferenceOps.swift:121-135 — q_proj output viewed [heads][2d]: head h's
// first d values are its query, the next d its gate.
void ho_split_query_gate(const double* combined, int heads, int d, double* query, double* gate) {
    for (int h = 0; h < heads; ++h) {
        for (int i = 0; i < d; ++i) {
            query[h * d + i] = combined[size_t(h) * 2 * d + i];
            gate[h * d + i] = combined[size_t(h) * 2 * d + d + i];
        }
    }
}

// Sources/HydraReference/QwenReferenceOps.swift:137-141 — out * sigmoid(gate).
void ho_apply_output_gate(const double* output, const double* gate, size_t n, double* out) {
    for (size_t i = 0; i < n; ++i) out[i] = output[i] * sigmoid(gate[i]);
}

// ---- The whole path for a batch of query rows --------------------------------------------------
//
// The attention part of ReferenceLayer.decode (Sources/HydraReference/ReferenceLayer.swift:152-183),
// Gemma4ReferenceLayer.forward (Gemma4ReferenceLayer.swift:146-162) and
// QwenReferenceAttentionLayer.forward (QwenReferenceLayer.swift:283-303), applied to `n_rows` query
// tokens that share one key/value history.
//
//   q         [n_rows][q_heads][d]   already normalised and rotated (float, holds bf16 values)
//   positions [n_rows]               absolute position of each query token
//   k, v      [history][kv_heads][d] the cache as the reference lays it out (float)
//   sinks     [q_heads] or null      null = no sink (Gemma, Qwen)
//   gate      [n_rows][q_heads][d] or null   Qwen's sigmoid output gate
//   window    0 = full causal; else keys [max(0, p - window + 1), p]
//   out       [n_rows][q_heads][d]   double
//
// Rows are independent and are spread over `threads` host threads.
//
// ho_attention_rows_blocks takes, besides, one entry per row: the position one past the end of the
// bidirectional block the row's token belongs to, or 0.  The reference's double-precision layers
// have no such mask; the rule is the Metal kernel's own loop bound, keyCount = max(blockEnd,
// position + 1) - start (Sources/HydraMetal/Shaders/batch.metal:340-352).
void ho_attention_rows_blocks(const float* q, const int64_t* positions, const int64_t* block_ends, int n_rows,
                              const float* k, const float* v, int q_heads, int kv_heads, int d, double sm_scale,
                              int window, const double* sinks, const float* gate, int threads, double* out);

void ho_attention_rows(const float* q, const int64_t* positions, int n_rows, const float* k,
                       const float* v, int q_heads, int kv_heads, int d, double sm_scale,
                       int window, const double* sinks, const float* gate, int threads,
                       double* out) {
    ho_attention_rows_blocks(q, positions, nullptr, n_rows, k, v, q_heads, kv_heads, d, sm_scale, window, sinks, gate,
                             threads, out);
}

void ho_attention_rows_blocks(const float* q, const int64_t* positions, const int64_t* block_ends, int n_rows,
                              const float* k, const float* v, int q_heads, int kv_heads, int d, double sm_scale,
                              int window, const double* sinks, const float* gate, int threads, double* out) {
    const int group = q_heads / kv_heads;
    parallel_for(n_rows * q_heads, threads, [&](int item) {
        const int row = item / q_heads;
        const int head = item % q_heads;
        const int kv_head = head / group;
        const int position = int(positions[row]);
        const int first = window > 0 ? std::max(0, position - window + 1) : 0;
        std::vector<double> logits;
        std::vector<double> query(size_t(d), 0.0);
        const float* qrow = q + (size_t(row) * q_heads + head) * d;
        for (int i = 0; i < d; ++i) query[size_t(i)] = double(qrow[i]);
        double* dest = out + (size_t(row) * q_heads + head) * d;
        int last = position;
        if (block_ends != nullptr && int(block_ends[row]) > position + 1) last = int(block_ends[row]) - 1;
        attend_row(query.data(), k + size_t(kv_head) * d, v + size_t(kv_head) * d,
                   ptrdiff_t(kv_heads) * d, first, last, d, sm_scale, sinks != nullptr,
                   sinks ? sinks[head] : 0.0, dest, logits);
        if (gate) {
            const float* grow = gate + (size_t(row) * q_heads + head) * d;
            for (int i = 0; i < d; ++i) dest[i] = dest[i] * sigmoid(double(grow[i]));
        }
    });
}

// The prologue of the path for a batch of tokens: per-head RMSNorm (optional, with or without a
// weight), then RoPE (optional), as Gemma4ReferenceLayer.keyValue
// (Sources/HydraReference/Gemma4ReferenceLayer.swift:223-248) and QwenReferenceAttentionLayer.forward
// (QwenReferenceLayer.swift:263-280) order them: norm before rotation, V normalised but never
// rotated.  The result is rounded to bf16 (BF16.swift:27-32) because that is what the cache and the
// kernels hold, and returned as float.
//
//   x         [n_rows][heads][d] float
//   positions [n_rows]
//   weight    [d] or null;  apply_norm = 0 skips the norm entirely
//   cos, sin  [n_rows][d/2] float tables for these rows, or null for no rotation
void ho_prepare_heads(const float* x, int n_rows, int heads, int d, int apply_norm,
                      const double* weight, double eps, const float* cosv, const float* sinv,
                      int round_bf16, int threads, float* out) {
    const int half = d / 2;
    parallel_for(n_rows, threads, [&](int row) {
        std::vector<double> a(size_t(d), 0.0), b(size_t(d), 0.0), c(size_t(half), 0.0), s(size_t(half), 0.0);
        for (int h = 0; h < heads; ++h) {
            const float* src = x + (size_t(row) * heads + h) * d;
            for (int i = 0; i < d; ++i) a[size_t(i)] = double(src[i]);
            if (apply_norm) {
                rms_norm(a.data(), weight, d, eps, false, b.data());
                a.swap(b);
            }
            if (cosv) {
                for (int i = 0; i < half; ++i) {
                    c[size_t(i)] = double(cosv[size_t(row) * half + i]);
                    s[size_t(i)] = double(sinv[size_t(row) * half + i]);
                }
                apply_rope(a.data(), d, c.data(), s.data(), b.data());
                a.swap(b);
            }
            float* dst = out + (size_t(row) * heads + h) * d;
            for (int i = 0; i < d; ++i) {
                const float f = float(a[size_t(i)]);
                dst[i] = round_bf16 ? bf16_to_float(bf16_from_float(f)) : f;
            }
        }
    });
}

}  // extern "C"
