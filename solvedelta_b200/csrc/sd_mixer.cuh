// Mixer glue around the chunked recurrence: depthwise causal conv4 + SiLU,
// the per-channel decay gate, and the sigmoid-gated RMSNorm, each with its
// reverse.  All are one pass over their operands (HBM bound); parameter
// gradients are reduced deterministically (per-CTA partials, then a column sum).
//
// Upstream counterparts: causallsso/model.py:110-164 (conv4 + SiLU with
// [B,D,3] state), model.py:375-390 (decay gate -exp(A) softplus(raw + bias)),
// causallsso/ops/norm_gate.py:19-43 (y = x rstd w sigmoid(gate)).
#pragma once
#include <type_traits>
#include "sd_common.cuh"

namespace sd {

constexpr int CONV_TT = 64;        // tokens per CTA of the conv kernels
constexpr int CONV_THREADS = 128;  // each thread owns two adjacent channels

struct ConvParams {
    int B, T, D;
    const __nv_bfloat16* x;  // [B,T,D] view: element strides sb, st, unit inner stride
    long long sb, st;
    const float* w;              // [D][4]
    const __nv_bfloat16* init;   // [B][D][3] or null
    __nv_bfloat16* y;            // [B,T,D] contiguous
    __nv_bfloat16* fin;          // [B][D][3] or null
    // backward
    const __nv_bfloat16* dy;     // [B,T,D] contiguous
    __nv_bfloat16* dx;           // [B,T,D] contiguous
    __nv_bfloat16* dinit;        // [B][D][3] or null
    float* dw_part;              // [B * tiles][D][4]
    // masks, one byte per (batch, token), either may be null (all valid / no reset)
    const unsigned char* valid;
    const unsigned char* reset;
};

// the fast reciprocal (2 ulp) instead of an IEEE division: these kernels are bound by instruction issue
__device__ __forceinline__ float silu_f(float z) { return __fdividef(z, 1.f + __expf(-z)); }
__device__ __forceinline__ float silu_grad_f(float z) {
    const float s = __fdividef(1.f, 1.f + __expf(-z));
    return s * (1.f + z * (1.f - s));
}

// input at (virtual) time t: the sequence for t >= 0, the carried state for -3 <= t < 0
__device__ __forceinline__ float2 conv_input(const ConvParams& p, int b, int t, int d, bool two) {
    float2 v = make_float2(0.f, 0.f);
    if (t >= 0) {
        if (t < p.T) {
            const __nv_bfloat16* row = p.x + b * p.sb + (long long)t * p.st + d;
            v.x = __bfloat162float(row[0]);
            if (two) v.y = __bfloat162float(row[1]);
        }
    } else if (p.init != nullptr) {
        const __nv_bfloat16* s = p.init + ((long long)b * p.D + d) * 3 + (t + 3);
        v.x = __bfloat162float(s[0]);
        if (two) v.y = __bfloat162float(s[3]);
    }
    return v;
}

// Two adjacent channels of one token of the sequence (t in [0, T)); PAIR: the pair is read /
// written as one 4-byte access (even strides and 4-byte aligned bases).
template <bool PAIR>
__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* row, bool two) {
    if (PAIR) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row));
    return make_float2(__bfloat162float(row[0]), two ? __bfloat162float(row[1]) : 0.f);
}
template <bool PAIR>
__device__ __forceinline__ void store_pair(__nv_bfloat16* row, bool two, float a, float b) {
    if (PAIR) {
        *reinterpret_cast<__nv_bfloat162*>(row) = __floats2bfloat162_rn(a, b);
    } else {
        row[0] = __float2bfloat16_rn(a);
        if (two) row[1] = __float2bfloat16_rn(b);
    }
}

// Ring of tokens in flight per thread (PAIR instantiations): every thread streams its own channel pair through
// shared memory with 4-byte cp.async copies, CONV_RING tokens ahead of the one it works on, so the walk along the
// sequence is not bound by one load latency per token.  A thread only ever touches its own ring column: no barrier.
constexpr int CONV_RING = 8;
__device__ __forceinline__ void conv_cp4(unsigned* smem, const __nv_bfloat16* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ float2 conv_ring_pair(unsigned raw) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw));
}

constexpr int CONV_BATCH = 4;      // forward: tokens whose loads are issued together
constexpr int CONV_BATCH_BWD = 1;  // reverse: more registers per token; batching cost occupancy and time

template <bool PAIR>
__global__ void __launch_bounds__(CONV_THREADS) k_conv4_silu_fwd(ConvParams p) {
    const int d = (blockIdx.x * CONV_THREADS + threadIdx.x) * 2;
    const int t0 = blockIdx.y * CONV_TT, b = blockIdx.z;
    if (d >= p.D) return;
    const bool two = d + 1 < p.D;
    float wa[4], wb[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        wa[j] = p.w[d * 4 + j];
        wb[j] = two ? p.w[(d + 1) * 4 + j] : 0.f;
    }
    float2 x0 = conv_input(p, b, t0 - 3, d, two), x1 = conv_input(p, b, t0 - 2, d, two),
           x2 = conv_input(p, b, t0 - 1, d, two);
    const int t1 = min(t0 + CONV_TT, p.T);
    const __nv_bfloat16* xin = p.x + b * p.sb + d;
    __nv_bfloat16* yout = p.y + (long long)b * p.T * p.D + d;
    if (PAIR) {
        __shared__ unsigned ring[CONV_RING][CONV_THREADS];
        auto issue = [&](int t) {
            if (t < t1) conv_cp4(&ring[(t - t0) % CONV_RING][threadIdx.x], xin + (long long)t * p.st);
            asm volatile("cp.async.commit_group;" ::);
        };
#pragma unroll
        for (int k = 0; k < CONV_RING; ++k) issue(t0 + k);
#pragma unroll 8
        for (int t = t0; t < t1; ++t) {
            asm volatile("cp.async.wait_group %0;" ::"n"(CONV_RING - 1));
            const float2 x3 = conv_ring_pair(ring[(t - t0) % CONV_RING][threadIdx.x]);
            issue(t + CONV_RING);
            const float za = wa[0] * x0.x + wa[1] * x1.x + wa[2] * x2.x + wa[3] * x3.x;
            const float zb = wb[0] * x0.y + wb[1] * x1.y + wb[2] * x2.y + wb[3] * x3.y;
            store_pair<PAIR>(yout + (long long)t * p.D, two, silu_f(za), silu_f(zb));
            x0 = x1; x1 = x2; x2 = x3;
        }
    } else
    for (int ts = t0; ts < t1; ts += CONV_BATCH) {
        float2 xs[CONV_BATCH];
#pragma unroll
        for (int k = 0; k < CONV_BATCH; ++k) {   // every token of a tile lies inside the sequence; only the tail is predicated
            xs[k] = make_float2(0.f, 0.f);
            if (ts + k < t1) xs[k] = load_pair<PAIR>(xin + (long long)(ts + k) * p.st, two);
        }
#pragma unroll
        for (int k = 0; k < CONV_BATCH; ++k) {
            if (ts + k < t1) {
                const float2 x3 = xs[k];
                const float za = wa[0] * x0.x + wa[1] * x1.x + wa[2] * x2.x + wa[3] * x3.x;
                const float zb = wb[0] * x0.y + wb[1] * x1.y + wb[2] * x2.y + wb[3] * x3.y;
                store_pair<PAIR>(yout + (long long)(ts + k) * p.D, two, silu_f(za), silu_f(zb));
                x0 = x1; x1 = x2; x2 = x3;
            }
        }
    }
    if (p.fin != nullptr && t1 == p.T) {
        // carried state = the last three inputs (the old state shows through when T < 3)
        __nv_bfloat16* s = p.fin + ((long long)b * p.D + d) * 3;
        s[0] = __float2bfloat16_rn(x0.x); s[1] = __float2bfloat16_rn(x1.x); s[2] = __float2bfloat16_rn(x2.x);
        if (two) {
            s[3] = __float2bfloat16_rn(x0.y); s[4] = __float2bfloat16_rn(x1.y); s[5] = __float2bfloat16_rn(x2.y);
        }
    }
}

template <bool PAIR>
__global__ void __launch_bounds__(CONV_THREADS) k_conv4_silu_bwd(ConvParams p) {
    const int d = (blockIdx.x * CONV_THREADS + threadIdx.x) * 2;
    const int t0 = blockIdx.y * CONV_TT, b = blockIdx.z;
    if (d >= p.D) return;
    const bool two = d + 1 < p.D;
    float wa[4], wb[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        wa[j] = p.w[d * 4 + j];
        wb[j] = two ? p.w[(d + 1) * 4 + j] : 0.f;
    }
    // sliding windows: x[t-3..t] and g[t-3..t] with g = dy * silu'(pre); g is zero outside [0,T).
    // dx[t-3] = w0 g[t] + w1 g[t-1] + w2 g[t-2] + w3 g[t-3]; tile 0 also emits t-3 < 0 (the state).
    // (g of tokens before the tile only feeds gradients that the previous tile emits)
    float2 x0 = conv_input(p, b, t0 - 3, d, two), x1 = conv_input(p, b, t0 - 2, d, two),
           x2 = conv_input(p, b, t0 - 1, d, two);
    float2 g0 = make_float2(0.f, 0.f), g1 = g0, g2 = g0;
    float dwa[4] = {0.f, 0.f, 0.f, 0.f}, dwb[4] = {0.f, 0.f, 0.f, 0.f};
    const int t_end = min(t0 + CONV_TT, p.T);
    const int t_last = min(t_end + 3, p.T);   // tokens past the tile still feed its last three gradients
    const __nv_bfloat16* xin = p.x + b * p.sb + d;
    const __nv_bfloat16* gin = p.dy + (long long)b * p.T * p.D + d;
    __nv_bfloat16* dxout = p.dx + (long long)b * p.T * p.D + d;
    if (PAIR) {
        __shared__ unsigned ring_x[CONV_RING][CONV_THREADS], ring_g[CONV_RING][CONV_THREADS];
        auto issue = [&](int t) {
            if (t < t_last) {
                conv_cp4(&ring_x[(t - t0) % CONV_RING][threadIdx.x], xin + (long long)t * p.st);
                conv_cp4(&ring_g[(t - t0) % CONV_RING][threadIdx.x], gin + (long long)t * p.D);
            }
            asm volatile("cp.async.commit_group;" ::);
        };
#pragma unroll
        for (int k = 0; k < CONV_RING; ++k) issue(t0 + k);
        // one token: INNER = a token of the tile with the whole tile's length behind it and three tokens of the tile
        // before it (every bound below holds, so none is tested)
        auto token = [&](int t, auto inner_tag) {
            constexpr bool INNER = decltype(inner_tag)::value;
            asm volatile("cp.async.wait_group %0;" ::"n"(CONV_RING - 1));
            float2 x3 = make_float2(0.f, 0.f), gy = x3;
            if (INNER || t < t_last) {
                x3 = conv_ring_pair(ring_x[(t - t0) % CONV_RING][threadIdx.x]);
                gy = conv_ring_pair(ring_g[(t - t0) % CONV_RING][threadIdx.x]);
            }
            issue(t + CONV_RING);
            float2 g3 = make_float2(0.f, 0.f);
            if (INNER || t < p.T) {
                const float za = wa[0] * x0.x + wa[1] * x1.x + wa[2] * x2.x + wa[3] * x3.x;
                const float zb = wb[0] * x0.y + wb[1] * x1.y + wb[2] * x2.y + wb[3] * x3.y;
                g3.x = gy.x * silu_grad_f(za);
                g3.y = gy.y * silu_grad_f(zb);
                if (INNER || t < t_end) {  // weight gradient: own tile only
                    dwa[0] += g3.x * x0.x; dwa[1] += g3.x * x1.x; dwa[2] += g3.x * x2.x; dwa[3] += g3.x * x3.x;
                    dwb[0] += g3.y * x0.y; dwb[1] += g3.y * x1.y; dwb[2] += g3.y * x2.y; dwb[3] += g3.y * x3.y;
                }
            }
            const int tq = t - 3;  // the input whose gradient is now complete
            const float da = wa[0] * g3.x + wa[1] * g2.x + wa[2] * g1.x + wa[3] * g0.x;
            const float db = wb[0] * g3.y + wb[1] * g2.y + wb[2] * g1.y + wb[3] * g0.y;
            if (INNER || (tq >= t0 && tq < t_end)) {
                store_pair<PAIR>(dxout + (long long)tq * p.D, two, da, db);
            } else if (tq < 0 && t0 == 0 && p.dinit != nullptr) {
                __nv_bfloat16* sd = p.dinit + ((long long)b * p.D + d) * 3 + (tq + 3);
                sd[0] = __float2bfloat16_rn(da);
                if (two) sd[3] = __float2bfloat16_rn(db);
            }
            x0 = x1; x1 = x2; x2 = x3;
            g0 = g1; g1 = g2; g2 = g3;
        };
        const int head_end = min(t0 + 3, t_end + 3);
        for (int t = t0; t < head_end; ++t) token(t, std::false_type{});
#pragma unroll 4
        for (int t = t0 + 3; t < t_end; ++t) token(t, std::true_type{});
        for (int t = max(t0 + 3, t_end); t < t_end + 3; ++t) token(t, std::false_type{});
    } else
    for (int ts = t0; ts < t_end + 3; ts += CONV_BATCH_BWD) {
        float2 xs[CONV_BATCH_BWD], gs[CONV_BATCH_BWD];
#pragma unroll
        for (int k = 0; k < CONV_BATCH_BWD; ++k) {
            xs[k] = make_float2(0.f, 0.f);
            gs[k] = make_float2(0.f, 0.f);
            if (ts + k < t_last) {
                xs[k] = load_pair<PAIR>(xin + (long long)(ts + k) * p.st, two);
                gs[k] = load_pair<PAIR>(gin + (long long)(ts + k) * p.D, two);
            }
        }
#pragma unroll
        for (int k = 0; k < CONV_BATCH_BWD; ++k) {
            const int t = ts + k;
            if (t < t_end + 3) {
                const float2 x3 = xs[k];
                float2 g3 = make_float2(0.f, 0.f);
                if (t < p.T) {
                    const float za = wa[0] * x0.x + wa[1] * x1.x + wa[2] * x2.x + wa[3] * x3.x;
                    const float zb = wb[0] * x0.y + wb[1] * x1.y + wb[2] * x2.y + wb[3] * x3.y;
                    g3.x = gs[k].x * silu_grad_f(za);
                    g3.y = gs[k].y * silu_grad_f(zb);
                    if (t < t_end) {  // weight gradient: own tile only
                        dwa[0] += g3.x * x0.x; dwa[1] += g3.x * x1.x; dwa[2] += g3.x * x2.x; dwa[3] += g3.x * x3.x;
                        dwb[0] += g3.y * x0.y; dwb[1] += g3.y * x1.y; dwb[2] += g3.y * x2.y; dwb[3] += g3.y * x3.y;
                    }
                }
                const int tq = t - 3;  // the input whose gradient is now complete
                const float da = wa[0] * g3.x + wa[1] * g2.x + wa[2] * g1.x + wa[3] * g0.x;
                const float db = wb[0] * g3.y + wb[1] * g2.y + wb[2] * g1.y + wb[3] * g0.y;
                if (tq >= t0 && tq < t_end) {
                    store_pair<PAIR>(dxout + (long long)tq * p.D, two, da, db);
                } else if (tq < 0 && t0 == 0 && p.dinit != nullptr) {
                    __nv_bfloat16* s = p.dinit + ((long long)b * p.D + d) * 3 + (tq + 3);
                    s[0] = __float2bfloat16_rn(da);
                    if (two) s[3] = __float2bfloat16_rn(db);
                }
                x0 = x1; x1 = x2; x2 = x3;
                g0 = g1; g1 = g2; g2 = g3;
            }
        }
    }
    float* part = p.dw_part + ((long long)(b * gridDim.y + blockIdx.y) * p.D + d) * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        part[j] = dwa[j];
        if (two) part[4 + j] = dwb[j];
    }
}

// ---- masked variants --------------------------------------------------------
// The masked token loop of causallsso/model.py:146-164 without repacking: an invalid token
// gives zero output and leaves the window untouched, a reset (on a valid token) empties the
// window first, so the three taps before a token are the last three valid inputs since the
// last reset (the carried state, oldest slots first, where the row has fewer).  The mask
// bytes of a tile are the same for every thread of a CTA, so all walks are uniform.
__device__ __forceinline__ bool conv_valid(const ConvParams& p, int b, int t) {
    return p.valid == nullptr || p.valid[(long long)b * p.T + t] != 0;
}
__device__ __forceinline__ bool conv_reset(const ConvParams& p, int b, int t) {
    return p.reset != nullptr && p.reset[(long long)b * p.T + t] != 0;
}
constexpr int CONV_NONE = -100;  // "no token" in a window slot

// Times (>= 0: tokens, -3..-1: slots of the carried state) of the three inputs before t0,
// newest first; CONV_NONE where a reset cut the window.
__device__ __forceinline__ void conv_window_before(const ConvParams& p, int b, int t0, int (&q)[3]) {
    int cnt = 0;
    bool cut = false;
    q[0] = q[1] = q[2] = CONV_NONE;
    for (int t = t0 - 1; t >= 0 && cnt < 3; --t) {
        if (!conv_valid(p, b, t)) continue;
        q[cnt++] = t;
        if (conv_reset(p, b, t)) {
            cut = true;
            break;
        }
    }
    if (!cut)
        for (int v = -1; cnt < 3; --v) q[cnt++] = v;
}
__device__ __forceinline__ float2 conv_input_at(const ConvParams& p, int b, int t, int d, bool two) {
    return t == CONV_NONE ? make_float2(0.f, 0.f) : conv_input(p, b, t, d, two);
}

template <bool PAIR>
__global__ void __launch_bounds__(CONV_THREADS) k_conv4_silu_fwd_masked(ConvParams p) {
    const int d = (blockIdx.x * CONV_THREADS + threadIdx.x) * 2;
    const int t0 = blockIdx.y * CONV_TT, b = blockIdx.z;
    if (d >= p.D) return;
    const bool two = d + 1 < p.D;
    float wa[4], wb[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        wa[j] = p.w[d * 4 + j];
        wb[j] = two ? p.w[(d + 1) * 4 + j] : 0.f;
    }
    int q[3];
    conv_window_before(p, b, t0, q);
    float2 x0 = conv_input_at(p, b, q[2], d, two), x1 = conv_input_at(p, b, q[1], d, two),
           x2 = conv_input_at(p, b, q[0], d, two);
    const int t1 = min(t0 + CONV_TT, p.T);
    const __nv_bfloat16* xin = p.x + b * p.sb + d;
    __nv_bfloat16* yout = p.y + (long long)b * p.T * p.D + d;
    for (int t = t0; t < t1; ++t) {
        if (!conv_valid(p, b, t)) {
            store_pair<PAIR>(yout + (long long)t * p.D, two, 0.f, 0.f);
            continue;
        }
        if (conv_reset(p, b, t)) x0 = x1 = x2 = make_float2(0.f, 0.f);
        const float2 x3 = load_pair<PAIR>(xin + (long long)t * p.st, two);
        const float za = wa[0] * x0.x + wa[1] * x1.x + wa[2] * x2.x + wa[3] * x3.x;
        const float zb = wb[0] * x0.y + wb[1] * x1.y + wb[2] * x2.y + wb[3] * x3.y;
        store_pair<PAIR>(yout + (long long)t * p.D, two, silu_f(za), silu_f(zb));
        x0 = x1; x1 = x2; x2 = x3;
    }
    if (p.fin != nullptr && t1 == p.T) {
        __nv_bfloat16* s = p.fin + ((long long)b * p.D + d) * 3;
        s[0] = __float2bfloat16_rn(x0.x); s[1] = __float2bfloat16_rn(x1.x); s[2] = __float2bfloat16_rn(x2.x);
        if (two) {
            s[3] = __float2bfloat16_rn(x0.y); s[4] = __float2bfloat16_rn(x1.y); s[5] = __float2bfloat16_rn(x2.y);
        }
    }
}

// Reverse of the masked loop.  Walking forward in time, the last three valid inputs are "pending":
// their gradients still collect terms from later tokens.  An input is complete when three valid
// tokens followed it, when a reset arrives, or at the end of the sequence.  A tile emits the
// gradients of its own tokens (and tile 0 those of the carried state), so it walks past its end
// until none of its own inputs is pending; weight gradients come from its own tokens only.
template <bool PAIR>
__global__ void __launch_bounds__(CONV_THREADS) k_conv4_silu_bwd_masked(ConvParams p) {
    const int d = (blockIdx.x * CONV_THREADS + threadIdx.x) * 2;
    const int t0 = blockIdx.y * CONV_TT, b = blockIdx.z;
    if (d >= p.D) return;
    const bool two = d + 1 < p.D;
    float wa[4], wb[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        wa[j] = p.w[d * 4 + j];
        wb[j] = two ? p.w[(d + 1) * 4 + j] : 0.f;
    }
    const int t_end = min(t0 + CONV_TT, p.T);
    const __nv_bfloat16* xin = p.x + b * p.sb + d;
    const __nv_bfloat16* gin = p.dy + (long long)b * p.T * p.D + d;
    __nv_bfloat16* dxout = p.dx + (long long)b * p.T * p.D + d;
    auto own = [&](int t) { return (t >= t0 && t < t_end) || (t < 0 && t >= -3 && t0 == 0 && p.dinit != nullptr); };
    auto emit = [&](int t, float2 a) {
        if (!own(t)) return;
        if (t >= 0) {
            store_pair<PAIR>(dxout + (long long)t * p.D, two, a.x, a.y);
        } else {
            __nv_bfloat16* s = p.dinit + ((long long)b * p.D + d) * 3 + (t + 3);
            s[0] = __float2bfloat16_rn(a.x);
            if (two) s[3] = __float2bfloat16_rn(a.y);
        }
    };
    int q[3];
    conv_window_before(p, b, t0, q);
    float2 x0 = conv_input_at(p, b, q[2], d, two), x1 = conv_input_at(p, b, q[1], d, two),
           x2 = conv_input_at(p, b, q[0], d, two);
    int i0 = q[2], i1 = q[1], i2 = q[0];  // pending inputs, oldest first (only own ones are ever emitted)
    float2 a0 = make_float2(0.f, 0.f), a1 = a0, a2 = a0;
    float dwa[4] = {0.f, 0.f, 0.f, 0.f}, dwb[4] = {0.f, 0.f, 0.f, 0.f};
    for (int t = t0; t < p.T; ++t) {
        if (t >= t_end && !own(i0) && !own(i1) && !own(i2)) break;
        if (!conv_valid(p, b, t)) {
            if (t < t_end) store_pair<PAIR>(dxout + (long long)t * p.D, two, 0.f, 0.f);
            continue;
        }
        if (conv_reset(p, b, t)) {
            emit(i0, a0); emit(i1, a1); emit(i2, a2);
            i0 = i1 = i2 = CONV_NONE;
            x0 = x1 = x2 = make_float2(0.f, 0.f);
        }
        const float2 x3 = load_pair<PAIR>(xin + (long long)t * p.st, two);
        const float2 gy = load_pair<PAIR>(gin + (long long)t * p.D, two);
        const float za = wa[0] * x0.x + wa[1] * x1.x + wa[2] * x2.x + wa[3] * x3.x;
        const float zb = wb[0] * x0.y + wb[1] * x1.y + wb[2] * x2.y + wb[3] * x3.y;
        const float2 g = make_float2(gy.x * silu_grad_f(za), gy.y * silu_grad_f(zb));
        if (t < t_end) {
            dwa[0] += g.x * x0.x; dwa[1] += g.x * x1.x; dwa[2] += g.x * x2.x; dwa[3] += g.x * x3.x;
            dwb[0] += g.y * x0.y; dwb[1] += g.y * x1.y; dwb[2] += g.y * x2.y; dwb[3] += g.y * x3.y;
        }
        a0.x += wa[0] * g.x; a0.y += wb[0] * g.y;
        a1.x += wa[1] * g.x; a1.y += wb[1] * g.y;
        a2.x += wa[2] * g.x; a2.y += wb[2] * g.y;
        emit(i0, a0);
        a0 = a1; i0 = i1;
        a1 = a2; i1 = i2;
        a2 = make_float2(wa[3] * g.x, wb[3] * g.y); i2 = t;
        x0 = x1; x1 = x2; x2 = x3;
    }
    // whatever is still pending saw the end of the sequence (entries that are not this tile's are skipped)
    emit(i0, a0); emit(i1, a1); emit(i2, a2);
    float* part = p.dw_part + ((long long)(b * gridDim.y + blockIdx.y) * p.D + d) * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        part[j] = dwa[j];
        if (two) part[4 + j] = dwb[j];
    }
}

// out[n] = sum_p partial[p][n]: deterministic column sum of per-CTA partials.  A CTA takes 32 columns with 32
// row lanes each (a lane adds every 32nd partial, eight loads in flight), then one thread per column adds the
// lanes in a fixed order.
constexpr int CSUM_COLS = 32, CSUM_LANES = 32;
__global__ void __launch_bounds__(CSUM_COLS * CSUM_LANES) k_column_sum(const float* part, int P, long long N, float* out) {
    __shared__ float s_lane[CSUM_LANES][CSUM_COLS + 1];
    const int cx = threadIdx.x % CSUM_COLS, ry = threadIdx.x / CSUM_COLS;
    const long long n = (long long)blockIdx.x * CSUM_COLS + cx;
    float acc = 0.f;
    if (n < N) {
#pragma unroll 8
        for (int q = ry; q < P; q += CSUM_LANES) acc += part[(long long)q * N + n];
    }
    s_lane[ry][cx] = acc;
    __syncthreads();
    if (ry == 0 && n < N) {
        float total = 0.f;
#pragma unroll
        for (int l = 0; l < CSUM_LANES; ++l) total += s_lane[l][cx];
        out[n] = total;
    }
}
inline void launch_column_sum(const float* part, int P, long long N, float* out, cudaStream_t stream) {
    k_column_sum<<<(unsigned)((N + CSUM_COLS - 1) / CSUM_COLS), CSUM_COLS * CSUM_LANES, 0, stream>>>(part, P, N, out);
}

// out[g] = sum_c in[g*width + c]: one warp per group, lanes stride the row, fixed shuffle tree.
__global__ void __launch_bounds__(32) k_group_sum(const float* in, int groups, int width, float* out) {
    const int g = blockIdx.x, lane = threadIdx.x;
    float acc = 0.f;
    for (int c = lane; c < width; c += 32) acc += in[(long long)g * width + c];
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
    if (lane == 0) out[g] = acc;
}

// ---- decay gate: log_decay = -exp(A[h]) * softplus(raw + bias[h][c]) ---------
struct GateParams {
    long long N;  // B*T rows
    int H, r;
    const __nv_bfloat16* raw;  // [N][H][r]
    const float* A;            // [H]
    const float* bias;         // [H][r]
    float* out;                // [N][H][r]
    const float* dout;         // backward
    __nv_bfloat16* draw;
    float* dA_part;            // [blocks][H]   (padded: one row of H*r + H per block, see host)
    float* dbias_part;         // [blocks][H][r]
    int rows_per_block;
};

// softplus(z) = max(z, 0) + log1p(exp(-|z|)) with the hardware exponential and logarithm: the argument of the
// logarithm lies in (1, 2], where its absolute error (about 4e-7) is below half an ulp of the BF16 input's own
// spacing by four orders of magnitude; below exp(-|z|) = 1e-3 two series terms replace it (relative error 3e-7).
__device__ __forceinline__ float softplus_fast(float z) {
    const float en = __expf(-fabsf(z));
    return fmaxf(z, 0.f) + (en < 1e-3f ? en * (1.f - 0.5f * en) : __logf(1.f + en));
}
// sigmoid(z) and softplus(z) from one exponential, en = exp(-|z|) in (0, 1]:
// softplus = max(z, 0) + log1p(en) (two series terms below 1e-3, where log(1 + en) would lose its digits).
// The reverse kernels use it: softplus only enters the sum for the rate gradient there.
__device__ __forceinline__ void sigmoid_softplus(float z, float& sig, float& sp) {
    const float en = __expf(-fabsf(z));
    const float inv = __fdividef(1.f, 1.f + en);
    sig = z >= 0.f ? inv : en * inv;
    sp = fmaxf(z, 0.f) + (en < 1e-3f ? en * (1.f - 0.5f * en) : __logf(1.f + en));
}

__global__ void k_kda_gate_fwd(GateParams p) {
    const long long total = p.N * p.H * p.r;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int hc = (int)(i % (p.H * p.r));
        const int h = hc / p.r;
        const float z = __bfloat162float(p.raw[i]) + p.bias[hc];
        p.out[i] = -__expf(p.A[h]) * softplus_fast(z);
    }
}

// Eight consecutive elements per thread (r % 8 == 0, 16-byte aligned operands).
__global__ void __launch_bounds__(256) k_kda_gate_fwd_v8(GateParams p) {
    const long long total8 = p.N * p.H * p.r / 8;
    const int HR = p.H * p.r;
    for (long long i8 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i8 < total8;
         i8 += (long long)gridDim.x * blockDim.x) {
        const long long i = i8 * 8;
        const int hc = (int)(i % HR);
        const float rate = -__expf(p.A[hc / p.r]);   // r % 8 == 0: the eight share a head
        const uint4 raw = *reinterpret_cast<const uint4*>(p.raw + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float4 b0 = *reinterpret_cast<const float4*>(p.bias + hc);
        const float4 b1 = *reinterpret_cast<const float4*>(p.bias + hc + 4);
        const float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]);
        const float2 f2 = __bfloat1622float2(h[2]), f3 = __bfloat1622float2(h[3]);
        *reinterpret_cast<float4*>(p.out + i) =
            make_float4(rate * softplus_fast(f0.x + b0.x), rate * softplus_fast(f0.y + b0.y),
                        rate * softplus_fast(f1.x + b0.z), rate * softplus_fast(f1.y + b0.w));
        *reinterpret_cast<float4*>(p.out + i + 4) =
            make_float4(rate * softplus_fast(f2.x + b1.x), rate * softplus_fast(f2.y + b1.y),
                        rate * softplus_fast(f3.x + b1.z), rate * softplus_fast(f3.y + b1.w));
    }
}

// blockIdx.x = block of rows, blockIdx.y = block of 256 (h, c) columns; one column per thread.
__global__ void __launch_bounds__(256) k_kda_gate_bwd(GateParams p) {
    const int hc = blockIdx.y * 256 + threadIdx.x, HR = p.H * p.r;
    if (hc >= HR) return;
    const int h = hc / p.r;
    const float rate = -__expf(p.A[h]), bias = p.bias[hc];
    const long long n0 = (long long)blockIdx.x * p.rows_per_block;
    const long long n1 = (n0 + p.rows_per_block < p.N) ? n0 + p.rows_per_block : p.N;
    float sum_b = 0.f, sum_a = 0.f;
    for (long long n = n0; n < n1; ++n) {
        const long long i = n * HR + hc;
        const float z = __bfloat162float(p.raw[i]) + bias;
        const float g = p.dout[i];
        float sig, sp;
        sigmoid_softplus(z, sig, sp);
        const float dz = g * rate * sig;
        p.draw[i] = __float2bfloat16_rn(dz);
        sum_b += dz;
        sum_a += g * rate * sp;  // d/dA of -exp(A) softplus = out
    }
    p.dbias_part[(long long)blockIdx.x * HR + hc] = sum_b;
    p.dA_part[(long long)blockIdx.x * HR + hc] = sum_a;  // summed over c on the host side of the ABI
}

// Eight consecutive columns per thread (H*r % 8 == 0, r % 8 == 0).  blockDim = 256 threads =
// cgb column groups x (256 / cgb) row lanes; blockIdx.x = block of rows, blockIdx.y = block of
// column groups.  Row lanes are summed through shared memory in a fixed order.
__global__ void __launch_bounds__(256) k_kda_gate_bwd_v8(GateParams p, int cgb) {
    __shared__ float s_part[256 * 16];
    const int HR = p.H * p.r;
    const int cg = threadIdx.x % cgb, lane = threadIdx.x / cgb, lanes = 256 / cgb;
    const int hc = (blockIdx.y * cgb + cg) * 8;
    const bool live = hc < HR;
    float sb[8], sa[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) sb[e] = sa[e] = 0.f;
    if (live) {
        const float rate = -__expf(p.A[hc / p.r]);
        const float4 b0 = *reinterpret_cast<const float4*>(p.bias + hc);
        const float4 b1 = *reinterpret_cast<const float4*>(p.bias + hc + 4);
        const float bias[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        const long long n0 = (long long)blockIdx.x * p.rows_per_block;
        const long long n1 = (n0 + p.rows_per_block < p.N) ? n0 + p.rows_per_block : p.N;
        // the next row's 48 bytes are requested before this row is worked on
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        float4 g0 = make_float4(0.f, 0.f, 0.f, 0.f), g1 = g0;
        long long n = n0 + lane;
        if (n < n1) {
            raw = *reinterpret_cast<const uint4*>(p.raw + n * HR + hc);
            g0 = *reinterpret_cast<const float4*>(p.dout + n * HR + hc);
            g1 = *reinterpret_cast<const float4*>(p.dout + n * HR + hc + 4);
        }
        for (; n < n1; n += lanes) {
            const long long i = n * HR + hc;
            const uint4 raw_c = raw;
            const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            if (n + lanes < n1) {
                const long long in = i + (long long)lanes * HR;
                raw = *reinterpret_cast<const uint4*>(p.raw + in);
                g0 = *reinterpret_cast<const float4*>(p.dout + in);
                g1 = *reinterpret_cast<const float4*>(p.dout + in + 4);
            }
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw_c);
            float dz[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float2 f = __bfloat1622float2(h[e >> 1]);
                const float z = ((e & 1) ? f.y : f.x) + bias[e];
                float sig, sp;
                sigmoid_softplus(z, sig, sp);
                dz[e] = g[e] * rate * sig;
                sb[e] += dz[e];
                sa[e] += g[e] * rate * sp;
            }
            uint4 outv;
            __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&outv);
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = __floats2bfloat162_rn(dz[2 * e], dz[2 * e + 1]);
            *reinterpret_cast<uint4*>(p.draw + i) = outv;
        }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        s_part[threadIdx.x * 16 + e] = sb[e];
        s_part[threadIdx.x * 16 + 8 + e] = sa[e];
    }
    __syncthreads();
    if (lane == 0 && live) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float tb = 0.f, ta = 0.f;
            for (int l = 0; l < lanes; ++l) {
                tb += s_part[(l * cgb + cg) * 16 + e];
                ta += s_part[(l * cgb + cg) * 16 + 8 + e];
            }
            p.dbias_part[(long long)blockIdx.x * HR + hc + e] = tb;
            p.dA_part[(long long)blockIdx.x * HR + hc + e] = ta;
        }
    }
}

// ---- sigmoid-gated RMSNorm over rows of width V <= 128 -------------------------
struct NormParams {
    long long N;  // rows
    int V;
    float eps;
    const __nv_bfloat16* x;
    const __nv_bfloat16* gate;
    const float* w;
    __nv_bfloat16* out;
    const __nv_bfloat16* dout;
    __nv_bfloat16* dx;
    __nv_bfloat16* dgate;
    float* dw_part;  // [blocks][V]
    int rows_per_block;
};

// Eight channels of a BF16 row starting at c0, as they lie (channels >= V and dead rows read as zero).  One
// 16-byte access when V is a multiple of eight (rows then start on 16-byte boundaries).
__device__ __forceinline__ uint4 norm_raw8(const __nv_bfloat16* row, int c0, int V, bool live) {
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if ((V & 7) == 0) {
        if (live && c0 < V) raw = *reinterpret_cast<const uint4*>(row + c0);
    } else {
        __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(&raw);
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (live && c0 + e < V) h[e] = row[c0 + e];
    }
    return raw;
}
__device__ __forceinline__ void norm_unpack8(const uint4& raw, float (&x)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        x[2 * e] = f.x;
        x[2 * e + 1] = f.y;
    }
}
__device__ __forceinline__ void norm_load8(const __nv_bfloat16* row, int c0, int V, bool live, float (&x)[8]) {
    norm_unpack8(norm_raw8(row, c0, V, live), x);
}
__device__ __forceinline__ void norm_store8(__nv_bfloat16* row, int c0, int V, bool live, const float (&x)[8]) {
    if (!live || c0 >= V) return;
    if ((V & 7) == 0) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
        *reinterpret_cast<uint4*>(row + c0) = raw;
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (c0 + e < V) row[c0 + e] = __float2bfloat16_rn(x[e]);
    }
}

// 16 lanes per row, 8 channels per lane; 256 threads = 16 rows at a time.
__global__ void __launch_bounds__(256) k_norm_gate_fwd(NormParams p) {
    const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
    for (long long base = (long long)blockIdx.x * 16; base < p.N; base += (long long)gridDim.x * 16) {
        const long long row = base + lr;
        const bool live = row < p.N;
        float x[8], g[8], y[8];
        float ss = 0.f;
        norm_load8(p.x + row * p.V, c0, p.V, live, x);
        norm_load8(p.gate + row * p.V, c0, p.V, live, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(x[e], x[e], ss);
        ss = row_sum16(ss);
        const float rstd = rsqrtf(ss / p.V + p.eps);
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = (c0 + e < p.V) ? x[e] * rstd * p.w[c0 + e] * sigmoidf_(g[e]) : 0.f;
        norm_store8(p.out + row * p.V, c0, p.V, live, y);
    }
}

__global__ void __launch_bounds__(256, 3) k_norm_gate_bwd(NormParams p) {
    __shared__ float s_dw[16][DP];
    const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
    float dw[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const long long n0 = (long long)blockIdx.x * p.rows_per_block;
    const long long n1 = (n0 + p.rows_per_block < p.N) ? n0 + p.rows_per_block : p.N;
    // the next row's three 16-byte pieces are requested before this row is worked on
    uint4 rx = norm_raw8(p.x + (n0 + lr) * p.V, c0, p.V, n0 + lr < n1);
    uint4 rg = norm_raw8(p.gate + (n0 + lr) * p.V, c0, p.V, n0 + lr < n1);
    uint4 rd = norm_raw8(p.dout + (n0 + lr) * p.V, c0, p.V, n0 + lr < n1);
    for (long long base = n0; base < n1; base += 16) {
        const long long row = base + lr;
        const bool live = row < n1;
        float x[8], g[8], dy[8];
        float ss = 0.f;
        norm_unpack8(rx, x);
        norm_unpack8(rg, g);
        norm_unpack8(rd, dy);
        {
            const long long nrow = row + 16;
            const bool nlive = nrow < n1;
            rx = norm_raw8(p.x + nrow * p.V, c0, p.V, nlive);
            rg = norm_raw8(p.gate + nrow * p.V, c0, p.V, nlive);
            rd = norm_raw8(p.dout + nrow * p.V, c0, p.V, nlive);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(x[e], x[e], ss);
        ss = row_sum16(ss);
        const float rstd = rsqrtf(ss / p.V + p.eps);
        // y = xn * w * s with xn = x rstd, s = sigmoid(g)
        float dxn[8], dot = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float s = sigmoidf_(g[e]);
            const float wv = (c0 + e < p.V) ? p.w[c0 + e] : 0.f;
            const float xn = x[e] * rstd;
            dw[e] += dy[e] * xn * s;
            dxn[e] = dy[e] * wv * s;
            dot = fmaf(dxn[e], xn, dot);
            g[e] = dy[e] * xn * wv * s * (1.f - s);  // d gate
        }
        dot = row_sum16(dot) / p.V;
        float dx[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) dx[e] = (dxn[e] - x[e] * rstd * dot) * rstd;
        norm_store8(p.dx + row * p.V, c0, p.V, live, dx);
        norm_store8(p.dgate + row * p.V, c0, p.V, live, g);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) s_dw[lr][c0 + e] = dw[e];
    __syncthreads();
    if (threadIdx.x < p.V) {
        float acc = 0.f;
#pragma unroll
        for (int q = 0; q < 16; ++q) acc += s_dw[q][threadIdx.x];
        p.dw_part[(long long)blockIdx.x * p.V + threadIdx.x] = acc;
    }
}

// ---- glue of the block around the mixer -----------------------------------------------------
// sum = x + delta (the residual stream, rounded to BF16 as the separate add stores it) and
// normed = sum rsqrt(mean(sum^2) + eps) w: the residual add and the RMSNorm that follows it
// (causallsso/modeling_solvedelta.py:230-255) in one pass.  k_add_rmsnorm: one CTA per row, any width (the few rows
// of a single-token step); k_add_rmsnorm_rows / k_add_rmsnorm_bwd below: one warp per row, forward and reverse.
struct AddNormParams {
    long long N;
    int D;
    float eps;
    const __nv_bfloat16 *x, *delta;   // delta may be null: sum = x, nothing is stored for it
    const float* w;
    __nv_bfloat16 *sum, *normed;
    // reverse pass: cotangents of the two outputs (dsum may be null), the one gradient x and delta share, partial
    // weight gradients [CTAs][D]
    const __nv_bfloat16 *dsum, *dnormed;
    __nv_bfloat16* dx;
    float* dw_part;
};

__global__ void __launch_bounds__(256) k_add_rmsnorm(AddNormParams p) {
    __shared__ float red[8];
    const long long row = blockIdx.x;
    const __nv_bfloat16* x = p.x + row * p.D;
    const __nv_bfloat16* d = p.delta + row * p.D;
    __nv_bfloat16* so = p.sum + row * p.D;
    float ss = 0.f;
    for (int c0 = threadIdx.x * 8; c0 < p.D; c0 += 256 * 8) {
        float a[8], b[8], s8[8];
        norm_load8(x, c0, p.D, true, a);
        norm_load8(d, c0, p.D, true, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            s8[e] = __bfloat162float(__float2bfloat16_rn(a[e] + b[e]));
            ss = fmaf(s8[e], s8[e], ss);
        }
        norm_store8(so, c0, p.D, true, s8);
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();   // also orders this thread's stores to `sum` before its reads below (same thread, same addresses)
    float tot = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) tot += red[w8];
    const float rstd = rsqrtf(tot / p.D + p.eps);
    __nv_bfloat16* no = p.normed + row * p.D;
    for (int c0 = threadIdx.x * 8; c0 < p.D; c0 += 256 * 8) {
        float s8[8], y[8];
        norm_load8(so, c0, p.D, true, s8);   // what this thread just wrote
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = (c0 + e < p.D) ? s8[e] * rstd * p.w[c0 + e] : 0.f;
        norm_store8(no, c0, p.D, true, y);
    }
}

// The same pair for rows of width D = 256 IT, one warp per row (a lane holds eight channels of every 256), used
// when D allows it; this is also the forward pass of training.  delta == nullptr: the norm alone.
constexpr int ADDNORM_WARPS = 4;
template <int IT>
__global__ void __launch_bounds__(32 * ADDNORM_WARPS) k_add_rmsnorm_rows(AddNormParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long stride = (long long)gridDim.x * ADDNORM_WARPS;
    for (long long row = (long long)blockIdx.x * ADDNORM_WARPS + warp; row < p.N; row += stride) {
        float s8[IT][8];
        float ss = 0.f;
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            const int c0 = it * 256 + lane * 8;
            norm_load8(p.x + row * p.D, c0, p.D, true, s8[it]);
            if (p.delta != nullptr) {
                float b[8];
                norm_load8(p.delta + row * p.D, c0, p.D, true, b);
#pragma unroll
                for (int e = 0; e < 8; ++e) s8[it][e] = __bfloat162float(__float2bfloat16_rn(s8[it][e] + b[e]));
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(s8[it][e], s8[it][e], ss);
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
        const float rstd = rsqrtf(ss / p.D + p.eps);
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            const int c0 = it * 256 + lane * 8;
            if (p.delta != nullptr) norm_store8(p.sum + row * p.D, c0, p.D, true, s8[it]);
            const float4 w0 = *reinterpret_cast<const float4*>(p.w + c0), w1 = *reinterpret_cast<const float4*>(p.w + c0 + 4);
            const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            float y[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = s8[it][e] * rstd * w[e];
            norm_store8(p.normed + row * p.D, c0, p.D, true, y);
        }
    }
}

// A 16-byte load that stays where it is written: the compiler otherwise sinks the loads of a row to their first
// use, which turns one memory phase per row into three.
__device__ __forceinline__ uint4 load16_pinned(const __nv_bfloat16* p) {
    uint4 r;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

// Reverse of the pair: with y = s rstd w and rstd = (mean(s^2) + eps)^-1/2,
//   ds = dsum + rstd (dn w - s rstd^2 mean(dn w s)),   dw = sum over rows of dn s rstd;
// ds is the gradient of x and of delta alike.  One warp per row; a CTA adds its warps' weight gradients in shared
// memory and leaves one partial row, which a column sum finishes.
template <int IT>
__global__ void __launch_bounds__(32 * ADDNORM_WARPS, 3) k_add_rmsnorm_bwd(AddNormParams p) {
    extern __shared__ float s_dw[];   // [ADDNORM_WARPS][D]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long stride = (long long)gridDim.x * ADDNORM_WARPS;
    // a warp's weight gradients live in its own row of shared memory (nobody else touches it before the barrier)
    float* my_dw = s_dw + warp * p.D;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
        *reinterpret_cast<float4*>(my_dw + it * 256 + lane * 8) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(my_dw + it * 256 + lane * 8 + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (long long row = (long long)blockIdx.x * ADDNORM_WARPS + warp; row < p.N; row += stride) {
        // every 16-byte piece of the row is requested at once and kept as it lies (BF16); the passes below unpack
        uint4 rs[IT], rn[IT], ru[IT];
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            const int c0 = it * 256 + lane * 8;
            rs[it] = load16_pinned(p.sum + row * p.D + c0);
            rn[it] = load16_pinned(p.dnormed + row * p.D + c0);
            ru[it] = p.dsum != nullptr ? load16_pinned(p.dsum + row * p.D + c0) : make_uint4(0u, 0u, 0u, 0u);
        }
        float ss = 0.f, dot = 0.f;
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            float s8[8];
            norm_unpack8(rs[it], s8);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(s8[e], s8[e], ss);
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
        const float rstd = rsqrtf(ss / p.D + p.eps);
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            const int c0 = it * 256 + lane * 8;
            const float4 w0 = *reinterpret_cast<const float4*>(p.w + c0), w1 = *reinterpret_cast<const float4*>(p.w + c0 + 4);
            const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            float s8[8], dn[8];
            norm_unpack8(rs[it], s8);
            norm_unpack8(rn[it], dn);
            float4 a0 = *reinterpret_cast<const float4*>(my_dw + c0), a1 = *reinterpret_cast<const float4*>(my_dw + c0 + 4);
            float dw[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                dw[e] = fmaf(dn[e] * rstd, s8[e], dw[e]);
                dot = fmaf(dn[e] * w[e], s8[e], dot);
            }
            *reinterpret_cast<float4*>(my_dw + c0) = make_float4(dw[0], dw[1], dw[2], dw[3]);
            *reinterpret_cast<float4*>(my_dw + c0 + 4) = make_float4(dw[4], dw[5], dw[6], dw[7]);
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, m);
        const float coef = dot * rstd * rstd / p.D;
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            const int c0 = it * 256 + lane * 8;
            const float4 w0 = *reinterpret_cast<const float4*>(p.w + c0), w1 = *reinterpret_cast<const float4*>(p.w + c0 + 4);
            const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            float s8[8], dn[8], up[8], ds[8];
            norm_unpack8(rs[it], s8);
            norm_unpack8(rn[it], dn);
            norm_unpack8(ru[it], up);
#pragma unroll
            for (int e = 0; e < 8; ++e) ds[e] = up[e] + rstd * (dn[e] * w[e] - s8[e] * coef);
            norm_store8(p.dx + row * p.D, c0, p.D, true, ds);
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < p.D; c += 32 * ADDNORM_WARPS) {
        float acc = 0.f;
#pragma unroll
        for (int q = 0; q < ADDNORM_WARPS; ++q) acc += s_dw[q * p.D + c];
        p.dw_part[(long long)blockIdx.x * p.D + c] = acc;
    }
}

// widths the one-warp-per-row kernels take: whole groups of 256 channels, at most eight of them
inline bool addnorm_rows_ok(int D) { return D % 256 == 0 && D <= 2048; }
// upper bound of the CTAs either kernel is launched with (sizes the partial weight gradients)
inline unsigned addnorm_blocks(long long rows) {
    long long blocks = (rows + ADDNORM_WARPS - 1) / ADDNORM_WARPS;
    return (unsigned)(blocks > 148 * 8 ? 148 * 8 : blocks);
}
// CTAs of `kernel` the whole device holds at once: a grid-stride kernel launched with more than that runs a partly
// filled last wave
template <class K>
inline unsigned resident_ctas(K kernel, int threads, size_t smem) {
    int per_sm = 0, sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem);
    return unsigned(per_sm < 1 ? 1 : per_sm) * unsigned(sms < 1 ? 1 : sms);
}
// returns the number of CTAs launched (= partial weight-gradient rows of the reverse kernel)
template <int IT>
inline unsigned launch_addnorm_rows(const AddNormParams& p, bool reverse, cudaStream_t stream) {
    const int threads = 32 * ADDNORM_WARPS;
    const size_t smem = reverse ? size_t(ADDNORM_WARPS) * p.D * sizeof(float) : 0;
    unsigned blocks = addnorm_blocks(p.N);
    const unsigned wave = reverse ? resident_ctas(k_add_rmsnorm_bwd<IT>, threads, smem)
                                  : resident_ctas(k_add_rmsnorm_rows<IT>, threads, smem);
    if (blocks > wave) blocks = wave;
    if (reverse) k_add_rmsnorm_bwd<IT><<<blocks, threads, smem, stream>>>(p);
    else k_add_rmsnorm_rows<IT><<<blocks, threads, smem, stream>>>(p);
    return blocks;
}
inline unsigned dispatch_addnorm_rows(const AddNormParams& p, bool reverse, cudaStream_t stream) {
    switch (p.D / 256) {
        case 1: return launch_addnorm_rows<1>(p, reverse, stream);
        case 2: return launch_addnorm_rows<2>(p, reverse, stream);
        case 3: return launch_addnorm_rows<3>(p, reverse, stream);
        case 4: return launch_addnorm_rows<4>(p, reverse, stream);
        case 5: return launch_addnorm_rows<5>(p, reverse, stream);
        case 6: return launch_addnorm_rows<6>(p, reverse, stream);
        case 7: return launch_addnorm_rows<7>(p, reverse, stream);
        default: return launch_addnorm_rows<8>(p, reverse, stream);
    }
}

// out = silu(gate) * value for rows [gate | value] of width 2 I (the gated MLP between its two
// projections, causallsso/modeling_solvedelta.py:68-101).
struct SwigluParams {
    long long N;
    int I;
    const __nv_bfloat16* in;   // [N][2 I]
    __nv_bfloat16* out;        // [N][I]
    const __nv_bfloat16* dout; // reverse pass: [N][I]
    __nv_bfloat16* din;        // reverse pass: [N][2 I]
};

__global__ void __launch_bounds__(256) k_swiglu(SwigluParams p) {
    const long long per_row = (p.I + 7) / 8, total = p.N * per_row;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long row = idx / per_row;
        const int c0 = (int)(idx - row * per_row) * 8;
        float g[8], v[8], y[8];
        norm_load8(p.in + row * 2 * p.I, c0, p.I, true, g);
        norm_load8(p.in + row * 2 * p.I + p.I, c0, p.I, true, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = silu_f(g[e]) * v[e];
        norm_store8(p.out + row * p.I, c0, p.I, true, y);
    }
}

// Reverse of k_swiglu: d gate = dout value silu'(gate), d value = dout silu(gate), written as one [gate | value] row.
__global__ void __launch_bounds__(256) k_swiglu_bwd(SwigluParams p) {
    const long long per_row = (p.I + 7) / 8, total = p.N * per_row;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long row = idx / per_row;
        const int c0 = (int)(idx - row * per_row) * 8;
        float g[8], v[8], d[8], dg[8], dv[8];
        norm_load8(p.in + row * 2 * p.I, c0, p.I, true, g);
        norm_load8(p.in + row * 2 * p.I + p.I, c0, p.I, true, v);
        norm_load8(p.dout + row * p.I, c0, p.I, true, d);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float sg = sigmoidf_(g[e]), act = g[e] * sg;
            dg[e] = d[e] * v[e] * (sg + act * (1.f - sg));
            dv[e] = d[e] * act;
        }
        norm_store8(p.din + row * 2 * p.I, c0, p.I, true, dg);
        norm_store8(p.din + row * 2 * p.I + p.I, c0, p.I, true, dv);
    }
}

// ---- gradient of the fused projection row, assembled from its slices ---------------------------------
// dst[row] = [piece 0 | piece 1 | ... | zeros]: every slice of the row (the conv's input gradient, the operator's
// four, the small projections') is a contiguous BF16 matrix of its own; one pass writes them side by side.  A
// thread owns one 16-byte group of the destination row and walks down the rows, four loads in flight.
constexpr int PACK_MAX_PIECES = 12;
struct PackRowsParams {
    long long N;
    int pieces, row_width;
    const __nv_bfloat16* src[PACK_MAX_PIECES];   // null: zeros
    int width[PACK_MAX_PIECES];
    __nv_bfloat16* dst;
};

__global__ void __launch_bounds__(256) k_pack_rows(PackRowsParams p) {
    const int c0 = (blockIdx.x * 256 + threadIdx.x) * 8;
    if (c0 >= p.row_width) return;
    const __nv_bfloat16* src = nullptr;
    int width = 0;
    {
        int off = 0;
        for (int k = 0; k < p.pieces; ++k) {
            if (c0 >= off && c0 < off + p.width[k]) {
                width = p.width[k];
                src = p.src[k] != nullptr ? p.src[k] + (c0 - off) : nullptr;
            }
            off += p.width[k];
        }
    }
    __nv_bfloat16* dst = p.dst + c0;
    const long long step = gridDim.y;
    long long row = blockIdx.y;
    if (src == nullptr) {
        for (; row < p.N; row += step) *reinterpret_cast<uint4*>(dst + row * p.row_width) = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    for (; row + 3 * step < p.N; row += 4 * step) {
        uint4 v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = *reinterpret_cast<const uint4*>(src + (row + k * step) * width);
#pragma unroll
        for (int k = 0; k < 4; ++k) *reinterpret_cast<uint4*>(dst + (row + k * step) * p.row_width) = v[k];
    }
    for (; row < p.N; row += step)
        *reinterpret_cast<uint4*>(dst + row * p.row_width) = *reinterpret_cast<const uint4*>(src + row * width);
}

// ---- cross entropy over BF16 logits (the FusedCrossEntropyLoss owner upstream calls, -------------------
// causallsso/modeling_solvedelta.py:469-470) ------------------------------------------------------------
// Forward: per row the log-sum-exp (kept for the reverse pass) and -log softmax(label) (0 for an ignored row), one
// read of the row.  Reverse: d logits = (softmax - onehot(label)) * coef with coef a device scalar (upstream
// gradient / token count), zeros for ignored rows.  One CTA per row; a thread takes 16-byte groups of the row.
struct CrossEntropyParams {
    long long N;
    int V;
    const __nv_bfloat16* logits;
    const long long* labels;
    long long ignore_index;
    float* lse;        // [N]
    float* row_loss;   // [N]
    const float* coef; // reverse: device scalar
    __nv_bfloat16* dlogits;
};

__device__ __forceinline__ float ce_block_reduce(float v, bool take_max, float* red) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, v, m);
        v = take_max ? fmaxf(v, o) : v + o;
    }
    __syncthreads();   // red is reused between calls
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) t = take_max ? fmaxf(t, red[w]) : t + red[w];
    return t;
}

__global__ void __launch_bounds__(256) k_cross_entropy_fwd(CrossEntropyParams p) {
    __shared__ float red[8];
    const long long row = blockIdx.x;
    const __nv_bfloat16* x = p.logits + row * p.V;
    const long long label = p.labels[row];
    // running maximum and sum of exp(x - maximum) per thread, merged at the end
    float mx = -INFINITY, sum = 0.f;
    for (int c0 = threadIdx.x * 8; c0 < p.V; c0 += 256 * 8) {
        float v[8];
        norm_load8(x, c0, p.V, true, v);
        float gm = mx;
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (c0 + e < p.V) gm = fmaxf(gm, v[e]);
        float add = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (c0 + e < p.V) add += __expf(v[e] - gm);
        sum = sum * __expf(mx - gm) + add;   // exp(-inf - finite) = 0 on the first group
        mx = gm;
    }
    const float top = ce_block_reduce(mx, true, red);
    const float total = ce_block_reduce(mx == -INFINITY ? 0.f : sum * __expf(mx - top), false, red);
    if (threadIdx.x == 0) {
        const float lse = top + __logf(total);
        p.lse[row] = lse;
        const bool live = label != p.ignore_index && label >= 0 && label < p.V;
        p.row_loss[row] = live ? lse - __bfloat162float(x[label]) : 0.f;
    }
}

__global__ void __launch_bounds__(256) k_cross_entropy_bwd(CrossEntropyParams p) {
    const long long row = blockIdx.x;
    const __nv_bfloat16* x = p.logits + row * p.V;
    __nv_bfloat16* d = p.dlogits + row * p.V;
    const long long label = p.labels[row];
    const bool live = label != p.ignore_index && label >= 0 && label < p.V;
    const float coef = live ? *p.coef : 0.f, lse = p.lse[row];
    for (int c0 = threadIdx.x * 8; c0 < p.V; c0 += 256 * 8) {
        float v[8], g[8];
        norm_load8(x, c0, p.V, true, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) g[e] = live ? (__expf(v[e] - lse) - (c0 + e == label ? 1.f : 0.f)) * coef : 0.f;
        norm_store8(d, c0, p.V, true, g);
    }
}

// ---- projections of a cached single-token step: y [M][N] = x [M][K] W^T (+ bias), M <= 4 ---------------
// At one to four rows a projection is a read of its weights: one warp per output column walks its weight row in
// 16-byte pieces (all loads of a row in flight at once) against the few input rows, FP32 accumulation, one
// shuffle reduction.  With `swiglu` a warp takes the gate row n and the value row n + N/2 and writes
// silu(gate) * value (the gated MLP's first projection and its activation in one launch).
constexpr int GEMV_MAX_ROWS = 4;
struct GemvParams {
    int M, N, K, swiglu;
    const __nv_bfloat16* x;
    long long x_stride;
    const __nv_bfloat16* W;
    const __nv_bfloat16* bias;
    __nv_bfloat16* y;
    long long y_stride;
};

__device__ __forceinline__ void gemv_row(const GemvParams& p, const __nv_bfloat16* w, int lane, float (&acc)[GEMV_MAX_ROWS]) {
#pragma unroll
    for (int m = 0; m < GEMV_MAX_ROWS; ++m) acc[m] = 0.f;
    // four 16-byte pieces of the weight row are requested together (pinned: the compiler would sink each load to its
    // use and leave one in flight per lane), then worked on
    for (int kb = lane * 8; kb < p.K; kb += 4 * 256) {
        uint4 raw[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
            raw[q] = kb + q * 256 < p.K ? load16_pinned(w + kb + q * 256) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k0 = kb + q * 256;
            if (k0 >= p.K) break;
            float wv[8];
            norm_unpack8(raw[q], wv);
#pragma unroll
            for (int m = 0; m < GEMV_MAX_ROWS; ++m) {
                if (m < p.M) {
                    float xv[8];
                    norm_unpack8(*reinterpret_cast<const uint4*>(p.x + m * p.x_stride + k0), xv);
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[m] = fmaf(wv[e], xv[e], acc[m]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < GEMV_MAX_ROWS; ++m)
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], s);
}

__global__ void __launch_bounds__(256) k_gemv(GemvParams p) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int outs = p.swiglu ? p.N / 2 : p.N;
    if (n >= outs) return;
    float a[GEMV_MAX_ROWS], b[GEMV_MAX_ROWS];
    gemv_row(p, p.W + (long long)n * p.K, lane, a);
    if (p.swiglu) gemv_row(p, p.W + (long long)(n + outs) * p.K, lane, b);
    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < GEMV_MAX_ROWS; ++m) {
            if (m < p.M) {
                float v = a[m] + (p.bias != nullptr ? __bfloat162float(p.bias[n]) : 0.f);
                if (p.swiglu) {
                    // both halves rounded to BF16 first, as the separate projection stores them
                    const float g = __bfloat162float(__float2bfloat16_rn(v));
                    const float u = __bfloat162float(__float2bfloat16_rn(
                        b[m] + (p.bias != nullptr ? __bfloat162float(p.bias[n + outs]) : 0.f)));
                    v = silu_f(g) * u;
                }
                p.y[m * p.y_stride + n] = __float2bfloat16_rn(v);
            }
        }
    }
}

}  // namespace sd
