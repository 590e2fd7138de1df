// Single-token recurrent step (T = 1, no gradient): one CTA per (batch, head)
// stream updates the FP32 cache (C, S) in place and emits one output row.
// The arithmetic is the token recurrence itself, in FP32.
#pragma once
#include "sd_common.cuh"

namespace sd {

struct DecodeParams {
    Geometry g;
    Operand u, h, q, k, v, er, wr, ld, gam;
    float *C, *S;
    void* y;
};

constexpr int DEC_THREADS = 128;

__device__ __forceinline__ float block_sum128(float v, float* red) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    return red[0] + red[1] + red[2] + red[3];
}

__global__ void __launch_bounds__(DEC_THREADS) k_decode_step(DecodeParams p) {
    __shared__ float s_uh[DP], s_kh[DP], s_alpha[DP], s_delta[DP], s_e[DP], s_chi[DP], s_d[DP];
    __shared__ float red[4];
    const int s = blockIdx.x, b = s / p.g.H, hh = s - b * p.g.H;
    const int r = p.g.r, V = p.g.V, tid = threadIdx.x;
    Chunk ch;
    ch.s = s; ch.c = 0; ch.b = b; ch.hh = hh; ch.t0 = 0; ch.nvalid = 1; ch.gi = s;
    ch.vm = 0ull; ch.rm = 0ull;
    const bool in_r = tid < r;
    float u = in_r ? __bfloat162float(row_bf16(p.u, ch, 0)[tid]) : 0.f;
    float k = in_r ? __bfloat162float(row_bf16(p.k, ch, 0)[tid]) : 0.f;
    float q = in_r ? __bfloat162float(row_bf16(p.q, ch, 0)[tid]) : 0.f;
    float hv = in_r ? __bfloat162float(row_bf16(p.h, ch, 0)[tid]) : 0.f;
    float er = in_r ? __bfloat162float(row_bf16(p.er, ch, 0)[tid]) : 0.f;
    float ld = in_r ? row_f32(p.ld, ch, 0)[tid] : 0.f;
    const float gamma = *row_f32(p.gam, ch, 0);
    float uh = u * rsqrtf(block_sum128(u * u, red) + 1e-24f);
    float kh = k * rsqrtf(block_sum128(k * k, red) + 1e-24f);
    float qh = q * rsqrtf(block_sum128(q * q, red) + 1e-24f);
    s_uh[tid] = uh;
    s_kh[tid] = kh;
    s_alpha[tid] = __expf(ld);
    __syncthreads();
    float* C = p.C + (long long)s * r * r;
    float* S = p.S + (long long)s * r * V;
    // residual against the old predictor: one warp per row of C
    {
        const int warp = tid >> 5, lane = tid & 31;
        for (int a = warp; a < r; a += DEC_THREADS / 32) {
            float acc = 0.f;
            for (int c = lane; c < r; c += 32) acc = fmaf(C[(long long)a * r + c], s_uh[c], acc);
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
            if (lane == 0) s_delta[a] = acc;
        }
    }
    __syncthreads();
    const float delta = in_r ? gamma * (hv - s_delta[tid]) : 0.f;
    __syncthreads();
    s_delta[tid] = delta;
    const float n2 = block_sum128(delta * delta, red);
    const float fs = RHO * rsqrtf(RHO * RHO + n2);
    const float phi = fs * delta;
    const float den = 1.f + block_sum128(phi * uh, red);
    const float bb = sigmoidf_(er) * kh;
    const float sb = block_sum128(uh * bb, red) / den;
    const float sq = block_sum128(uh * qh, red) / den;
    s_e[tid] = bb - phi * sb;
    s_chi[tid] = qh - phi * sq;
    // right-decay + rank-one write of C, and d = k^ + C_new^T k^ (thread = column)
    float dcol = kh;
    if (in_r) {
        const float al = s_alpha[tid];
        for (int a = 0; a < r; ++a) {
            float cn = fmaf(C[(long long)a * r + tid], al, s_delta[a] * uh);
            C[(long long)a * r + tid] = cn;
            dcol = fmaf(cn, s_kh[a], dcol);
        }
    }
    s_d[tid] = in_r ? dcol : 0.f;
    __syncthreads();
    // memory: decay rows, read along e, write along d, read along chi (thread = value column)
    if (tid < V) {
        float pred = 0.f;
        for (int c = 0; c < r; ++c) pred = fmaf(s_alpha[c] * S[(long long)c * V + tid], s_e[c], pred);
        const float wr = __bfloat162float(row_bf16(p.wr, ch, 0)[tid]);
        const float vv = __bfloat162float(row_bf16(p.v, ch, 0)[tid]);
        const float w = sigmoidf_(wr) * vv - pred;
        float out = 0.f;
        for (int c = 0; c < r; ++c) {
            float sn = fmaf(s_alpha[c], S[(long long)c * V + tid], s_d[c] * w);
            S[(long long)c * V + tid] = sn;
            out = fmaf(sn, s_chi[c], out);
        }
        reinterpret_cast<__nv_bfloat16*>(p.y)[(long long)s * V + tid] = __float2bfloat16_rn(out);
    }
}

}  // namespace sd
