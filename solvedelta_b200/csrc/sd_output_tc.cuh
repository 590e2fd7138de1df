// The output contraction of a chunk on the fifth-generation tensor cores:
//     y = Xg S_c + Aqd Z~        (chunk_dplr_fwd_kernel_o upstream, causallsso/ops/residual_frame/common_left_o_fwd.py:101-135)
// with Xg = chi exp(G) [CL][DP], S_c the chunk-entry state [DP][DP], Aqd the causal pair matrix [CL][CL] and
// Z~ [CL][DP], all BF16 panels in HBM.  One CTA per (stream, chunk):
//   * seven tiled TMA loads (cp.async.bulk.tensor.3d with the 128-byte swizzle, bytes counted on one
//     mbarrier) land the panels in shared memory as tiles of 64 contiguous elements (128-byte rows): Xg and
//     Aqd, contiguous along the contraction, as K-major tiles [rows][64]; S_c and Z~, contiguous along the
//     output column, as MN-major tiles [contraction rows][64 columns];
//   * one thread issues twelve tcgen05.mma.kind::f16 (M = 128 of which 64 rows are real, N = 128, K = 16),
//     eight over the state rows and four over the chunk's tokens, into one FP32 accumulator in tensor memory
//     (128 of the 512 columns), then tcgen05.commit onto a second mbarrier;
//   * the four warps that own tensor-memory lanes 0..63 read the accumulator back (tcgen05.ld), round to
//     BF16 and store the output rows with 16-byte stores (exact zeros for masked tokens).
// 73 KB of shared memory and 128 tensor-memory columns per CTA: three CTAs share an SM, so one CTA's loads
// overlap another's contraction and epilogue.  Rows 64..127 of the A operands alias whatever follows them in
// shared memory and only feed accumulator lanes nobody reads.
//
// Both waits are bounded; a wait that runs out stores 6 (panels never landed) or 7 (contraction never
// completed) in the device fault word, the CTA writes nothing and still frees its tensor memory.
#pragma once
#include "sd_forward.cuh"
#include "sd_scan_tc.cuh"

namespace sd {

constexpr int OUT_TC_THREADS = 256;
constexpr unsigned OUT_XG_BYTES = CL * DP * 2;    // two K tiles [CL][64]
constexpr unsigned OUT_AQD_BYTES = CL * CL * 2;   // one K tile [CL][64]
constexpr unsigned OUT_S_BYTES = DP * DP * 2;     // two N tiles [DP][64]
constexpr unsigned OUT_ZT_BYTES = CL * DP * 2;    // two N tiles [CL][64]
constexpr unsigned OUT_TC_PANEL_BYTES = OUT_XG_BYTES + OUT_AQD_BYTES + OUT_S_BYTES + OUT_ZT_BYTES;
constexpr size_t OUTPUT_TC_SMEM = OUT_TC_PANEL_BYTES + 1024 + 128;   // + room to align the tiles to 1024 bytes
// the padded A operands (M = 128) reach 64 rows = 8 KB past their tiles: Xg into Aqd, Aqd into S
static_assert(OUT_AQD_BYTES >= 8192 && OUT_S_BYTES >= 8192, "padded operand rows leave the allocation");
static_assert(3 * (OUTPUT_TC_SMEM + 1024) <= 228 * 1024, "three output CTAs per SM");

// FP32 accumulator, BF16 operands, A K-major, B MN-major, M = 128
__device__ __forceinline__ unsigned out_tc_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(n >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void out_tc_mma(unsigned d_tmem, unsigned long long da, unsigned long long db,
                                           unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
// one tile: 64 columns starting at `col`, every row of the panel of `task`
__device__ __forceinline__ void out_tc_load(unsigned char* sm, const CUtensorMap* map, int col, int task, unsigned bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            tc_smem(sm)),
        "l"(reinterpret_cast<unsigned long long>(map)), "r"(col), "r"(0), "r"(task), "r"(bar)
        : "memory");
}
// Shared-memory matrix descriptor for the 128-byte swizzle (tile base 1024-byte aligned).  K-major: rows of 128
// bytes, 8-row groups 1024 bytes apart (sbo), a K step of 16 elements advances the start address by 32 bytes.
// MN-major: lbo = bytes between 64-column tiles, sbo = 1024 (8 contraction rows), a K step advances 2048 bytes.
__device__ __forceinline__ unsigned long long out_tc_desc(unsigned addr, unsigned lbo, unsigned sbo) {
    return tc_desc(addr, lbo, sbo) | (2ull << 61);
}

template <bool MASKED>
__global__ void __launch_bounds__(OUT_TC_THREADS, 3)
k_output_fwd_tc(FwdParams p, const __grid_constant__ CUtensorMap xg_map, const __grid_constant__ CUtensorMap aqd_map,
                const __grid_constant__ CUtensorMap s_map, const __grid_constant__ CUtensorMap zt_map, int* fault) {
    extern __shared__ __align__(16) unsigned char osm_raw[];
    unsigned char* osm = osm_raw + ((1024u - (tc_smem(osm_raw) & 1023u)) & 1023u);   // swizzled tiles: 1024-byte aligned
    unsigned char* sXg = osm;
    unsigned char* sAqd = sXg + OUT_XG_BYTES;
    unsigned char* sS = sAqd + OUT_AQD_BYTES;
    unsigned char* sZt = sS + OUT_S_BYTES;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sZt + OUT_ZT_BYTES);
    unsigned* s_tmem = reinterpret_cast<unsigned*>(bars + 2);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const ChunkT<MASKED> ch = chunk_of<MASKED>(p.g, blockIdx.x);
    const int V = p.g.V;
    int ph = 0;
    SD_PHASE(p.g, ph);

    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&bars[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&bars[1])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(s_tmem)), "r"(128));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tbase = *s_tmem;
    const unsigned bar_load = tc_smem(&bars[0]), bar_mma = tc_smem(&bars[1]);
    SD_PHASE(p.g, ph);

    if (tid == 0) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_load), "r"(OUT_TC_PANEL_BYTES)
                     : "memory");
        const int task = (int)ch.gi;
        out_tc_load(sXg, &xg_map, 0, task, bar_load);
        out_tc_load(sXg + OUT_XG_BYTES / 2, &xg_map, 64, task, bar_load);
        out_tc_load(sAqd, &aqd_map, 0, task, bar_load);
        out_tc_load(sS, &s_map, 0, task, bar_load);
        out_tc_load(sS + OUT_S_BYTES / 2, &s_map, 64, task, bar_load);
        out_tc_load(sZt, &zt_map, 0, task, bar_load);
        out_tc_load(sZt + OUT_ZT_BYTES / 2, &zt_map, 64, task, bar_load);
    }
    bool alive = tc_wait(bar_load, 0);
    if (!alive) atomicExch(fault, 6);
    SD_PHASE(p.g, ph);
    if (tid == 0 && alive) {
        tc_fence_after();
        const unsigned idesc = out_tc_idesc(DP);
        // Xg: two K tiles of 64 channels (8 KB each);  S: two N tiles of 64 value columns (16 KB each), 16 state rows
        // per step
#pragma unroll
        for (int ks = 0; ks < DP / 16; ++ks)
            out_tc_mma(tbase, out_tc_desc(tc_smem(sXg) + (ks / 4) * (OUT_XG_BYTES / 2) + (ks % 4) * 32, 16, 1024),
                       out_tc_desc(tc_smem(sS) + ks * 2048, OUT_S_BYTES / 2, 1024), idesc, ks > 0 ? 1u : 0u);
        // Aqd: one K tile over the chunk's tokens;  Z~: two N tiles (8 KB each)
#pragma unroll
        for (int ks = 0; ks < CL / 16; ++ks)
            out_tc_mma(tbase, out_tc_desc(tc_smem(sAqd) + ks * 32, 16, 1024),
                       out_tc_desc(tc_smem(sZt) + ks * 2048, OUT_ZT_BYTES / 2, 1024), idesc, 1u);
        tc_commit(bar_mma);
    }
    // lanes 0..63 hold the chunk's rows: warps 0, 1, 4, 5 read them back, 64 columns each
    const int quarter = warp & 3, half = warp >> 2;
    if (quarter < 2) {
        bool done = alive && tc_wait(bar_mma, 0);
        done = __all_sync(0xffffffffu, done);   // the reads below are warp-wide (sync.aligned)
        if (alive && !done && lane == 0) atomicExch(fault, 7);
        tc_fence_after();
        SD_PHASE(p.g, ph);
        if (done) {
            const int i = quarter * 32 + lane;
            const bool live = i < ch.nvalid, ok = ch.ok(i);
            __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(p.y) +
                                 (((long long)ch.b * p.g.T + ch.t0 + (live ? i : 0)) * p.g.H + ch.hh) * (long long)V;
            const bool vec = (V & 7) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 15) == 0;
#pragma unroll
            for (int part = 0; part < 2; ++part) {
                const int j0 = half * 64 + part * 32;
                float acc[32];
                tc_ld32(tbase + ((unsigned)(quarter * 32) << 16) + j0, acc);
                tc_wait_ld();
                if (!live) continue;   // rows past the end of the sequence
#pragma unroll
                for (int j8 = 0; j8 < 32; j8 += 8) {
                    const int j = j0 + j8;
                    if (j >= V) break;
                    if (vec) {
                        uint4 w;
                        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            h2[e] = ok ? __floats2bfloat162_rn(acc[j8 + 2 * e], acc[j8 + 2 * e + 1])
                                       : __floats2bfloat162_rn(0.f, 0.f);
                        *reinterpret_cast<uint4*>(row + j) = w;
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (j + e < V) row[j + e] = __float2bfloat16_rn(ok ? acc[j8 + e] : 0.f);
                    }
                }
            }
        }
    }
    SD_PHASE(p.g, ph);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(128));
}

}  // namespace sd
