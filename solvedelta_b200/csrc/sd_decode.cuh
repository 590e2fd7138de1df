// Single-token recurrent step (T = 1, no gradient): one CTA per (batch, head) stream updates the FP32 cache
// (C, S) in place and emits one output row.  The arithmetic is the token recurrence itself, in FP32.
//
// The step is pure state traffic (2 x 64 KiB read and written per stream at r = V = 128), so the kernel is
// built around moving each state exactly once: both states stream into shared memory with 16-byte cp.async
// copies issued up front (S lands behind the predictor phase), every phase works on the shared copies with
// all 512 threads (four threads per row for the row dots, four row quarters per column for the column
// sums), and each state goes back with 16-byte stores as soon as its phase is done.
// Upstream counterparts: _predictor_recurrent_kernel, _relative_recurrent_sources_kernel and the fused
// recurrent DPLR step (causallsso/ops/residual_frame/recurrent.py:33-98,188-327).
#pragma once
#include "sd_bf16.cuh"
#include "sd_common.cuh"
#include "sd_mixer.cuh"

namespace sd {

struct DecodeParams {
    Geometry g;
    Operand u, h, q, k, v, er, wr, ld, gam;
    float *C, *S;
    void* y;
};

// The mixer glue of a cached single-token step, computed inside the decode kernel (k_decode_step<true>):
// q, k, v = SiLU(conv4) of the projection row against the carried three-token window, which is advanced in
// place (causallsso/model.py:146-164 at T = 1); log decay = -exp(A[h]) softplus(raw + bias) (model.py:383-390);
// geometry rate = sigmoid(raw + bias) (model.py:391-394).  The operands q, k, v, ld, gam of DecodeParams are
// then unused.
struct MixerDecode {
    const __nv_bfloat16* qkv;       // conv input of the token: [B] rows of D = 2 H r + H V channels (q | k | v)
    long long qkv_sb;               // elements between batch rows
    const float* conv_w;            // [D][4], tap 3 multiplies the current token
    __nv_bfloat16* conv_state;      // [B][D][3], oldest first; in/out
    const __nv_bfloat16* decay_raw; // [B][H*r]
    long long decay_sb;
    const float* log_rate;          // [H]
    const float* decay_bias;        // [H*r]
    const __nv_bfloat16* geom_raw;  // [B][H]
    long long geom_sb;
    const float* geom_bias;         // [H]
    // optional (norm_w != null): the sigmoid-gated RMSNorm of the output row (causallsso/ops/norm_gate.py:19-43)
    const float* norm_w;            // [V]
    float norm_eps;
    const __nv_bfloat16* gate;      // [B][H*V]
    long long gate_sb;
    // optional (decay_w / gate_w != null): the two small projections in front of the gates are taken here too,
    // raw = BF16(W hidden (+ bias)) with W [H*r][G] / [H*V][G] (causallsso/model.py:369-374); decay_raw / gate
    // above are then unused
    int G;
    const __nv_bfloat16 *decay_hidden, *decay_w;   // [B][G] (row stride dh_sb), [H*r][G]
    long long dh_sb;
    const __nv_bfloat16 *gate_hidden, *gate_w, *gate_b;   // [B][G], [H*V][G], [H*V] or null
    long long gh_sb;
};

// Partial dot of up to 64 weights (BF16, 16-byte aligned) with `hidden`: every piece of the weight row is requested
// before any is used (pinned loads: a loop of load-then-multiply waits for memory once per piece).
__device__ __forceinline__ float decode_row_dot_pinned(const __nv_bfloat16* w, const float* hidden, int span) {
    uint4 raw[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) raw[q] = q * 8 < span ? load16_pinned(w + q * 8) : make_uint4(0u, 0u, 0u, 0u);
    float acc = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        if (q * 8 < span) {
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[q]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(h2[e]);
                acc = fmaf(f.x, hidden[q * 8 + 2 * e], fmaf(f.y, hidden[q * 8 + 2 * e + 1], acc));
            }
        }
    }
    return acc;
}

// one conv channel of the token: output (rounded to BF16 as the separate conv kernel stores it), window advanced
__device__ __forceinline__ float decode_conv_channel(const MixerDecode& m, int b, int D, int chn) {
    __nv_bfloat16* st = m.conv_state + ((long long)b * D + chn) * 3;
    const __nv_bfloat16 b0 = st[0], b1 = st[1], b2 = st[2], b3 = m.qkv[(long long)b * m.qkv_sb + chn];
    const float* w = m.conv_w + chn * 4;
    const float z = w[0] * __bfloat162float(b0) + w[1] * __bfloat162float(b1) + w[2] * __bfloat162float(b2) +
                    w[3] * __bfloat162float(b3);
    st[0] = b1; st[1] = b2; st[2] = b3;
    return __bfloat162float(__float2bfloat16_rn(silu_f(z)));
}

constexpr int DEC_THREADS = 512;
constexpr int DEC_LD = DP + 4;   // row pitch of a shared state (floats)
constexpr size_t DECODE_SMEM = (size_t(2) * DP * DEC_LD + 12 * DP + 96) * sizeof(float);

// sum over the first DP threads' values (the others pass 0), returned to every thread
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_THREADS / 32; ++w) t += red[w];
    return t;
}

// N sums at once (one pair of barriers for all of them); red holds [N][16] floats
template <int N>
__device__ __forceinline__ void block_sum_n(float (&v)[N], float* red) {
#pragma unroll
    for (int n = 0; n < N; ++n)
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) v[n] += __shfl_xor_sync(0xffffffffu, v[n], m);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) {
#pragma unroll
        for (int n = 0; n < N; ++n) red[n * (DEC_THREADS / 32) + (threadIdx.x >> 5)] = v[n];
    }
    __syncthreads();
#pragma unroll
    for (int n = 0; n < N; ++n) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_THREADS / 32; ++w) t += red[n * (DEC_THREADS / 32) + w];
        v[n] = t;
    }
}

// [rows][cols] FP32 state in global memory (row pitch `cols`) -> shared [DP][DEC_LD], zero padded
__device__ __forceinline__ void decode_state_in(float* sm, const float* g, int rows, int cols, bool vec) {
    for (int idx = threadIdx.x; idx < DP * (DP / 4); idx += DEC_THREADS) {
        const int a = idx >> 5, c4 = (idx & 31) << 2;
        float* dst = sm + a * DEC_LD + c4;
        if (vec) {
            cp16_zfill(dst, g + (long long)(a < rows ? a : 0) * cols + (c4 < cols ? c4 : 0), a < rows && c4 < cols);
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) dst[e] = (a < rows && c4 + e < cols) ? g[(long long)a * cols + c4 + e] : 0.f;
        }
    }
}
__device__ __forceinline__ void decode_state_out(float* g, const float* sm, int rows, int cols, bool vec) {
    for (int idx = threadIdx.x; idx < DP * (DP / 4); idx += DEC_THREADS) {
        const int a = idx >> 5, c4 = (idx & 31) << 2;
        if (a >= rows || c4 >= cols) continue;
        const float* src = sm + a * DEC_LD + c4;
        if (vec) {
            *reinterpret_cast<float4*>(g + (long long)a * cols + c4) = *reinterpret_cast<const float4*>(src);
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (c4 + e < cols) g[(long long)a * cols + c4 + e] = src[e];
        }
    }
}

template <bool MIXER>
__global__ void __launch_bounds__(DEC_THREADS, 1) k_decode_step(DecodeParams p, MixerDecode mix) {
    extern __shared__ __align__(16) float dsm[];
    float* sC = dsm;                       // [DP][DEC_LD]
    float* sS = sC + DP * DEC_LD;          // [DP][DEC_LD]
    float* s_uh = sS + DP * DEC_LD;
    float* s_kh = s_uh + DP;
    float* s_alpha = s_kh + DP;
    float* s_delta = s_alpha + DP;
    float* s_e = s_delta + DP;
    float* s_chi = s_e + DP;
    float* s_d = s_chi + DP;
    float* s_w = s_d + DP;
    float* s_part = s_w + DP;              // [4][DP] partial column sums
    float* red = s_part + 4 * DP;          // [5][16] (block_sum_n)
    const int s = blockIdx.x, b = s / p.g.H, hh = s - b * p.g.H;
    const int r = p.g.r, V = p.g.V, tid = threadIdx.x;
    Chunk ch;
    ch.s = s; ch.c = 0; ch.b = b; ch.hh = hh; ch.t0 = 0; ch.nvalid = 1; ch.gi = s;
    ch.vm = 0ull; ch.rm = 0ull;
    float* C = p.C + (long long)s * r * r;
    float* S = p.S + (long long)s * r * V;
    // 16-byte moves need rows that start on 16-byte boundaries
    const bool vecC = (r & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0;
    const bool vecS = (V & 3) == 0 && (reinterpret_cast<uintptr_t>(p.S) & 15) == 0;
    decode_state_in(sC, C, r, r, vecC);
    cp_commit();
    decode_state_in(sS, S, r, V, vecS);
    cp_commit();

    const bool in_r = tid < r;     // threads 0..r-1 carry the token's channel values
    float u = in_r ? __bfloat162float(row_bf16(p.u, ch, 0)[tid]) : 0.f;
    float hv = in_r ? __bfloat162float(row_bf16(p.h, ch, 0)[tid]) : 0.f;
    float er = in_r ? __bfloat162float(row_bf16(p.er, ch, 0)[tid]) : 0.f;
    float k = 0.f, q = 0.f, ld = 0.f, gamma, v_mix = 0.f;
    float gate_mix = 0.f;   // raw output gate of this thread's value channel (fused projection)
    if (MIXER) {
        const int H = p.g.H, D = 2 * H * r + H * V;
        float decay_raw_mix = 0.f;
        if (mix.decay_w != nullptr) {   // kernel-uniform: the two small projections
            float* s_hid = s_part;      // [2][G]: free until the predictor phase
            for (int j = tid; j < 2 * mix.G; j += DEC_THREADS) {
                const bool second = j >= mix.G;
                const int jj = second ? j - mix.G : j;
                s_hid[j] = __bfloat162float(second ? mix.gate_hidden[(long long)b * mix.gh_sb + jj]
                                                   : mix.decay_hidden[(long long)b * mix.dh_sb + jj]);
            }
            __syncthreads();
            {
                // two threads per output (r decay rows, then V gate rows: all 512 threads at r = V = 128), each half
                // of the row's G weights; the pair adds up through a shuffle and leaves the BF16-rounded value in
                // shared memory for the thread that owns the channel
                float* s_proj = s_part + 2 * mix.G;   // [r + V], behind the hidden rows (G <= 128)
                const int row2 = tid >> 1, half = tid & 1, span = mix.G / 2;
                const bool is_gate = row2 >= r;
                const int rr = is_gate ? row2 - r : row2;
                const bool live = rr < (is_gate ? V : r);
                float part = 0.f;
                if (live) {
                    const __nv_bfloat16* w = is_gate ? mix.gate_w + (long long)(hh * V + rr) * mix.G
                                                     : mix.decay_w + (long long)(hh * r + rr) * mix.G;
                    part = decode_row_dot_pinned(w + half * span, s_hid + (is_gate ? mix.G : 0) + half * span, span);
                }
                part += __shfl_xor_sync(0xffffffffu, part, 1);
                if (live && half == 0) {
                    const float bias = is_gate && mix.gate_b ? __bfloat162float(mix.gate_b[hh * V + rr]) : 0.f;
                    s_proj[row2] = __bfloat162float(__float2bfloat16_rn(part + bias));
                }
                __syncthreads();
                if (in_r) decay_raw_mix = s_proj[tid];
                if (tid < V) gate_mix = s_proj[r + tid];
            }
            __syncthreads();   // s_part is reused below
        }
        if (in_r) {
            q = decode_conv_channel(mix, b, D, hh * r + tid);
            k = decode_conv_channel(mix, b, D, H * r + hh * r + tid);
            const int hc = hh * r + tid;
            const float raw = mix.decay_w != nullptr ? decay_raw_mix
                                                     : __bfloat162float(mix.decay_raw[(long long)b * mix.decay_sb + hc]);
            const float z = raw + mix.decay_bias[hc];
            ld = -__expf(mix.log_rate[hh]) * softplus_fast(z);
        }
        if (tid < V) v_mix = decode_conv_channel(mix, b, D, 2 * H * r + hh * V + tid);
        const float graw = __bfloat162float(mix.geom_raw[(long long)b * mix.geom_sb + hh]) + mix.geom_bias[hh];
        gamma = 1.f / (1.f + __expf(-graw));
    } else {
        k = in_r ? __bfloat162float(row_bf16(p.k, ch, 0)[tid]) : 0.f;
        q = in_r ? __bfloat162float(row_bf16(p.q, ch, 0)[tid]) : 0.f;
        ld = in_r ? row_f32(p.ld, ch, 0)[tid] : 0.f;
        gamma = *row_f32(p.gam, ch, 0);
    }
    // the three norms and the two dot products that only need them, in one reduction
    const float se = sigmoidf_(er);
    float sums[5] = {u * u, k * k, q * q, u * se * k, u * q};
    block_sum_n<5>(sums, red);
    const float rs_u = rsqrtf(sums[0] + 1e-24f), rs_k = rsqrtf(sums[1] + 1e-24f), rs_q = rsqrtf(sums[2] + 1e-24f);
    const float uh = u * rs_u, kh = k * rs_k, qh = q * rs_q;
    const float dot_ub = sums[3] * rs_u * rs_k, dot_uq = sums[4] * rs_u * rs_q;   // u^ . (sigma(e) k^),  u^ . q^
    if (tid < DP) {
        s_uh[tid] = uh;
        s_kh[tid] = kh;
        s_alpha[tid] = __expf(ld);
    }
    cp_wait<1>();      // C has landed
    __syncthreads();
    // residual against the old predictor: four threads per row of C, 32 columns each
    {
        const int a = tid >> 2, q4 = (tid & 3) * 32;
        float acc = 0.f;
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
            const float4 cv = *reinterpret_cast<const float4*>(sC + a * DEC_LD + q4 + c);
            const float4 uv = *reinterpret_cast<const float4*>(s_uh + q4 + c);
            acc = fmaf(cv.x, uv.x, fmaf(cv.y, uv.y, fmaf(cv.z, uv.z, fmaf(cv.w, uv.w, acc))));
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        if ((tid & 3) == 0) s_delta[a] = acc;
    }
    __syncthreads();
    const float delta = in_r ? gamma * (hv - s_delta[tid]) : 0.f;
    __syncthreads();
    if (tid < DP) s_delta[tid] = delta;
    float two[2] = {delta * delta, delta * uh};
    block_sum_n<2>(two, red);
    const float n2 = two[0];
    const float fs = RHO * rsqrtf(RHO * RHO + n2);
    const float phi = fs * delta;
    const float den = 1.f + fs * two[1];
    const float bb = se * kh;
    const float sb = dot_ub / den;
    const float sq = dot_uq / den;
    if (tid < DP) {
        s_e[tid] = bb - phi * sb;
        s_chi[tid] = qh - phi * sq;
    }
    __syncthreads();
    // right-decay + rank-one write of C, and d = k^ + C_new^T k^ : thread = (column, quarter of the rows)
    const int col = tid & (DP - 1), a0 = (tid >> 7) * 32;
    {
        const float al = s_alpha[col], uc = s_uh[col];
        float part = 0.f;
#pragma unroll 8
        for (int a = a0; a < a0 + 32; ++a) {
            const float cn = fmaf(sC[a * DEC_LD + col], al, s_delta[a] * uc);
            sC[a * DEC_LD + col] = cn;
            part = fmaf(cn, s_kh[a], part);
        }
        s_part[(tid >> 7) * DP + col] = part;
    }
    cp_wait<0>();      // S has landed
    __syncthreads();
    decode_state_out(C, sC, r, r, vecC);
    if (tid < DP) s_d[tid] = (tid < r) ? kh + (s_part[tid] + s_part[DP + tid]) + (s_part[2 * DP + tid] + s_part[3 * DP + tid]) : 0.f;
    // memory: prediction along e on the decayed rows (thread = (value column, quarter of the rows))
    {
        float part = 0.f;
#pragma unroll 8
        for (int c = a0; c < a0 + 32; ++c) part = fmaf(s_alpha[c] * sS[c * DEC_LD + col], s_e[c], part);
        __syncthreads();   // the partial sums of d have been read
        s_part[(tid >> 7) * DP + col] = part;
    }
    __syncthreads();
    if (tid < DP) {
        float w = 0.f;
        if (tid < V) {
            const float wr = __bfloat162float(row_bf16(p.wr, ch, 0)[tid]);
            const float vv = MIXER ? v_mix : __bfloat162float(row_bf16(p.v, ch, 0)[tid]);
            w = sigmoidf_(wr) * vv - ((s_part[tid] + s_part[DP + tid]) + (s_part[2 * DP + tid] + s_part[3 * DP + tid]));
        }
        s_w[tid] = w;
    }
    __syncthreads();
    // decay rows, write along d, read along chi
    {
        const float w = s_w[col];
        float part = 0.f;
#pragma unroll 8
        for (int c = a0; c < a0 + 32; ++c) {
            const float sn = fmaf(s_alpha[c], sS[c * DEC_LD + col], s_d[c] * w);
            sS[c * DEC_LD + col] = sn;
            part = fmaf(sn, s_chi[c], part);
        }
        s_part[(tid >> 7) * DP + col] = part;
    }
    __syncthreads();
    decode_state_out(S, sS, r, V, vecS);
    float yv = 0.f;   // the output element of this thread, rounded to BF16 as the operator returns it
    if (tid < V)
        yv = __bfloat162float(__float2bfloat16_rn((s_part[tid] + s_part[DP + tid]) +
                                                  (s_part[2 * DP + tid] + s_part[3 * DP + tid])));
    if (MIXER && mix.norm_w != nullptr) {   // kernel-uniform
        const float rstd = rsqrtf(block_sum(yv * yv, red) / V + mix.norm_eps);
        if (tid < V) {
            const float g = mix.gate_w != nullptr ? gate_mix
                                                  : __bfloat162float(mix.gate[(long long)b * mix.gate_sb + hh * V + tid]);
            yv = yv * rstd * mix.norm_w[tid] * sigmoidf_(g);
        }
    }
    if (tid < V) reinterpret_cast<__nv_bfloat16*>(p.y)[(long long)s * V + tid] = __float2bfloat16_rn(yv);
}

}  // namespace sd
