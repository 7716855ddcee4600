// Fused NF4 dequant-GEMV, staged variant: packed weights and absmax travel HBM -> shared memory
// by TMA (cp.async.bulk.tensor.2d, completion on an mbarrier, no multicast): one request moves a
// box of 16 (or 8) weight rows x one K segment, so DRAM sees long sequential bursts, nothing
// passes through the L1 tag stage and the data in flight lives in a shared-memory ring instead of
// registers.  The box is 32 bytes wider than the segment (and the absmax box 4 floats wider): that
// makes the row pitch in shared memory 32 mod 128 bytes, which keeps the fragment loads free of
// bank conflicts without a swizzle mode.
//
// One CTA per SM: 16 compute warps + 1 producer warp.  A stage of the ring holds one tile of 16
// weight rows x SB 64-blocks (SB <= 32: up to 1 KB of codes per row) plus the SB absmax values
// of each row.  Compute warp w owns blocks 2w and 2w+1 of every stage (K is split over the warps),
// builds the A fragments of mma.sync.m16n8k16 from the packed bytes with the conflict-free lookup
// table (see nf4_gemv_common.cuh), multiplies them with the activation fragments (B operand, up to
// 8 activation rows per column tile) and folds the 4 accumulators of a 64-block into the running
// sum with that block's fp32 absmax.  Rows are processed in groups of TG tiles so an activation
// fragment is fetched once per (group, K segment); at the end of a group the 16 partial sums per
// output meet in shared memory, in fixed order, and leave as bf16/fp16.
//
// Every wait on an mbarrier is bounded (wall-clock limit); on a time-out the CTA records an error
// code in a device word (read it with nf4_b200_device_error), stops waiting and runs to its end.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>
#include <type_traits>

#include "nf4_gemv_common.cuh"

namespace nf4 {

constexpr int SG_MAX_STAGES = 8;
constexpr int SG_PF_ROWS = 32;          // rows of the next launch's weights a CTA prefetches into L2 (one per producer lane; measured
                                        // in the decode chain: 16-48 rows 1.2 % faster than 64, 128 rows 7 % slower, none 0.3 % faster than 64)
constexpr int SG_PF_ROW_BYTES = 2048;   // ... and bytes of each row (4096 weights)
constexpr unsigned long long SG_WAIT_LIMIT_NS = 200ull * 1000 * 1000;   // 0.2 s per wait

__device__ unsigned int g_gemv_error[4];   // [0] first error code, [1] block, [2] stage, [3] count

struct alignas(64) StagedParams {
    CUtensorMap wmap16, wmap8;   // packed codes viewed as uint64 [N][K/16], boxes of 16 and 8 rows
    CUtensorMap amap16, amap8;   // absmax fp32 [N][K/64], boxes of 16 and 8 rows
    const void* x;
    const uint8_t* packed;
    const float* absmax;     // fp32 [N*KB]; with double quantization: the uint8 indices (absmax_u8) instead
    // double-quantized absmax (template flag DQ): absmax = fma(code256[u8], scale2[block / 256], *offset)
    const uint8_t* absmax_u8;
    const float* scale2;
    const float* offset;
    const float* code256;
    const float* code16;
    const void* bias;
    const void* residual;   // optional [M][N], added after the bias (may alias y)
    void* y;
    int M, N, K, KB;
    int SB;          // 64-blocks per stage (divides KB, multiple of 4, <= 32)
    int nseg;        // KB / SB
    int NS;          // ring stages
    int RS;          // bytes between weight rows inside a stage (SB*32 + 32)
    int AS;          // bytes between absmax rows inside a stage (SB*4 + 16)
    int stage_bytes; // 16*RS + 16*AS
    int x_staged;    // activations are copied to shared memory
    int x_stride;    // bytes between staged activation rows (2K + 16; 4K + 16 with the SiLU prologue)
    int prologue;    // 0: none; 1: x <- rmsnorm(x) * norm_w; 2: x <- silu(x[:, :K]) * x[:, K:2K]  (x is [M][2K])
    const void* norm_w;   // [K], prologue 1
    float eps;
    int epilogue;    // 0: y[m][n]; 1: rows come in (gate, up) pairs and y[m][n/2] = silu(gate) * up;
                     // 2: rows [0, N/2) are gate, [N/2, N) up: a tile is 8 gate rows + the 8 matching up rows
    // offsets from the start of dynamic shared memory
    int off_bars, off_part, off_x;
    int off_c256;    // DQ: the 256-entry table of the second quantization (1 KB)
    int h_base, h_rem;   // halves of 8 rows per CTA: h_base, plus one for the first h_rem CTAs
    // L2 prefetch of the next launch's weights (null: none): same row split, applied to its N
    const uint8_t* pf_packed;
    const float* pf_absmax;
    int pf_N, pf_row_bytes, pf_am_row_bytes, pf_h_base, pf_h_rem;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Programmatic dependent launch: a kernel launched with the stream-serialization attribute may start
// while its predecessor is still running; `griddep_wait` blocks until the predecessor grid has
// finished and its writes are visible (no-op for a normal launch), `griddep_launch` lets the
// successor start early.  Everything before the wait may only touch weights and the kernel's own
// shared memory.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}

// Bounded wait.  The hot path is a plain poll of the barrier; only a wait that has already lasted thousands
// of polls starts reading the timer and the CTA's abort flag (returns at once when the CTA has given up).
__device__ __noinline__ void mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, int stage) {
    if (*abort_flag) return;
    const unsigned long long t0 = global_ns();
    while (true) {
        for (int spin = 0; spin < 256; ++spin)
            if (mbar_try_wait(bar, parity)) return;
        if (*abort_flag) return;
        if (global_ns() - t0 > SG_WAIT_LIMIT_NS) {
            *abort_flag = 1;
            if (atomicCAS(&g_gemv_error[0], 0u, (unsigned)code) == 0u) {
                g_gemv_error[1] = blockIdx.x;
                g_gemv_error[2] = (unsigned)stage;
            }
            atomicAdd(&g_gemv_error[3], 1u);
            return;
        }
    }
}
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, int stage) {
#pragma unroll 1
    for (int spin = 0; spin < 4096; ++spin)
        if (mbar_try_wait(bar, parity)) return;
    mbar_wait_slow(bar, parity, abort_flag, code, stage);
}

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds32f(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// One stage of one warp: BPW 64-blocks of a 16-row tile.  Per block: 16 table lookups, 4 chained
// MMAs per column tile (the chains of different blocks interleave), one scaling by the block's
// absmax.  HALF: rows 8..15 of the tile do not exist (their fragment registers stay zero).
// The BPW blocks of a warp are adjacent, so their absmax values (or, with double quantization, their uint8
// indices) come with one load per row.  DQ: sc[0/1] are the second-level scales of this lane's two rows -- a
// stage never straddles a group of 256 first-level blocks -- fetched by the caller before it waited for the
// stage; c256 is the shared-memory table, dq_off the offset.
template <int BPW>
__device__ __forceinline__ void load_absmax(uint32_t addr, float (&am)[BPW]) {
    if constexpr (BPW == 2) {
        asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(am[0]), "=f"(am[1]) : "r"(addr));
    } else {
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(am[0]), "=f"(am[1]), "=f"(am[2]), "=f"(am[3]) : "r"(addr));
    }
}
template <int BPW>
__device__ __forceinline__ void load_absmax_dq(uint32_t addr, uint32_t c256, float scale, float dq_off, float (&am)[BPW]) {
    uint32_t bytes;
    if constexpr (BPW == 2) asm volatile("ld.shared.u16 %0, [%1];" : "=r"(bytes) : "r"(addr));
    else asm volatile("ld.shared.u32 %0, [%1];" : "=r"(bytes) : "r"(addr));
#pragma unroll
    for (int bi = 0; bi < BPW; ++bi) am[bi] = fmaf(lds32f(c256 + 4u * ((bytes >> (8 * bi)) & 0xffu)), scale, dq_off);
}

template <typename T, int NT, int BPW, bool HALF, bool DQ>
__device__ __forceinline__ void stage_compute(uint32_t sbase, const uint32_t (&a_off)[BPW], uint32_t am_off,
                                              uint32_t rs8, uint32_t as8, uint32_t window_lane,
                                              const uint32_t (&xf)[BPW][NT][8], float (&acc)[NT][4],
                                              const float (&sc)[2], uint32_t c256, float dq_off) {
    uint2 wa[BPW], wb[BPW];
    float ama[BPW], amb[BPW];
#pragma unroll
    for (int bi = 0; bi < BPW; ++bi) {
        wa[bi] = lds64(sbase + a_off[bi]);
        if (!HALF) wb[bi] = lds64(sbase + a_off[bi] + rs8);
    }
    if (DQ) {
        load_absmax_dq<BPW>(sbase + am_off, c256, sc[0], dq_off, ama);
        if (!HALF) load_absmax_dq<BPW>(sbase + am_off + as8, c256, sc[1], dq_off, amb);
    } else {
        load_absmax<BPW>(sbase + am_off, ama);
        if (!HALF) load_absmax<BPW>(sbase + am_off + as8, amb);
    }
    float tmp[BPW][NT][4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
#pragma unroll
        for (int bi = 0; bi < BPW; ++bi) {
            const uint32_t va = (t < 2) ? wa[bi].x : wa[bi].y;
            uint32_t a[4];
            a[1] = 0u;
            a[3] = 0u;
            if (t & 1) {
                a[0] = lut_lookup<2>(va, window_lane);
                a[2] = lut_lookup<3>(va, window_lane);
            } else {
                a[0] = lut_lookup<0>(va, window_lane);
                a[2] = lut_lookup<1>(va, window_lane);
            }
            if (!HALF) {
                const uint32_t vb = (t < 2) ? wb[bi].x : wb[bi].y;
                if (t & 1) {
                    a[1] = lut_lookup<2>(vb, window_lane);
                    a[3] = lut_lookup<3>(vb, window_lane);
                } else {
                    a[1] = lut_lookup<0>(vb, window_lane);
                    a[3] = lut_lookup<1>(vb, window_lane);
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                if (t == 0) Mma<T>::run0(tmp[bi][nt], a, xf[bi][nt][0], xf[bi][nt][1]);
                else Mma<T>::acc(tmp[bi][nt], a, xf[bi][nt][2 * t], xf[bi][nt][2 * t + 1]);
            }
        }
    }
#pragma unroll
    for (int bi = 0; bi < BPW; ++bi)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            acc[nt][0] = fmaf(tmp[bi][nt][0], ama[bi], acc[nt][0]);
            acc[nt][1] = fmaf(tmp[bi][nt][1], ama[bi], acc[nt][1]);
            if (!HALF) {
                acc[nt][2] = fmaf(tmp[bi][nt][2], amb[bi], acc[nt][2]);
                acc[nt][3] = fmaf(tmp[bi][nt][3], amb[bi], acc[nt][3]);
            }
        }
}

// GU: epilogue 2 (SwiGLU over [gate rows; up rows]).  A template flag, not a run-time test: the extra producer
// and finishing code measurably slowed the plain kernel (about 3 % of a decode step) when it was compiled in.
template <typename T, int NT, int TG, int CW, bool DQ, bool GU>
__global__ void __launch_bounds__((CW + 1) * 32, 1) gemv_staged_kernel(const __grid_constant__ StagedParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr int BPW = 32 / CW;          // 64-blocks of a stage per warp
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int g = lane >> 2;
    const int q = lane & 3;

    const uint32_t s0 = smem_u32(smem);
    const uint32_t lut_base = (s0 + LUT_WINDOW - 1) & ~(uint32_t)(LUT_WINDOW - 1);
    uint8_t* const lut_ptr = smem + (lut_base - s0);
    const uint32_t ring_u32 = lut_base + LUT_WINDOW;
    uint64_t* const bars = reinterpret_cast<uint64_t*>(smem + p.off_bars);   // full[NS], empty[NS], xbar
    volatile int* const abort_flag = reinterpret_cast<volatile int*>(smem + p.off_bars + (2 * SG_MAX_STAGES + 1) * 8);
    float* const part = reinterpret_cast<float*>(smem + p.off_part);
    const uint32_t xs_u32 = s0 + (uint32_t)p.off_x;
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + SG_MAX_STAGES * 8, xbar = full0 + 2 * SG_MAX_STAGES * 8;

    // rows are dealt out in halves of 8: a CTA owns [8*h0, 8*h1); full 16-row tiles first, then at
    // most one half tile
    // (epilogue 2: the halves count gate rows; every half is a full tile with its 8 up rows)
    const int bid = (int)blockIdx.x;
    constexpr bool split_gu = GU;
    const int n_own = split_gu ? (p.N >> 1) : p.N;      // rows that are dealt out
    const int tile_rows = split_gu ? 8 : 16;            // ... and how many of them one tile covers
    const int h0 = bid * p.h_base + min(bid, p.h_rem);
    const int h1 = h0 + p.h_base + (bid < p.h_rem ? 1 : 0);
    const int r0 = h0 * 8;
    const int r1 = min(h1 * 8, n_own);
    const int nhalves = h1 - h0;
    const int nfull = split_gu ? nhalves : (nhalves >> 1);
    const int ntiles = split_gu ? nhalves : nfull + (nhalves & 1);

    if (s0 > 2048u) {   // the host-side map assumes the dynamic region starts within 2 KB of the window
        if (tid == 0 && atomicCAS(&g_gemv_error[0], 0u, 4u) == 0u) g_gemv_error[1] = blockIdx.x;
        return;
    }
    // The start of the kernel is a chain of latencies (first weight boxes, the level table's source, the
    // activations), so they are all put in flight before anybody waits: the producer's first lane arms
    // the barriers, signals that (a non-blocking arrival at named barrier 2) and starts issuing boxes;
    // the compute warps fetch the levels, build the table and start the activation copy meanwhile and
    // then wait on barrier 2, which makes the armed barriers and the table visible to all of them.
    const float level = warp < CW ? __ldg(p.code16 + (lane & 15)) : 0.0f;

    // Both roles walk the same schedule: groups of up to TG full tiles, then the half tile alone;
    // inside a group: for every K segment, every tile of the group -> one stage each.
    if (warp == CW) {
        // ------------------------------- producer warp --------------------------------------
        // The weights do not depend on the previous kernel, so this warp never waits for it; the
        // activations are fetched by compute warp 0 once the predecessor grid has finished.
        if (lane == 0) {
            for (int s = 0; s < p.NS; ++s) {
                mbar_init(full0 + s * 8, 1);
                mbar_init(empty0 + s * 8, CW);
            }
            *abort_flag = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        asm volatile("bar.arrive 2, %0;" ::"n"((CW + 1) * 32) : "memory");
        griddep_launch();
        int stage = 0, slot = 0;
        uint32_t parity = 0;
        for (int tile0 = 0; tile0 < ntiles;) {
            const bool half = tile0 >= nfull;
            const int nt_here = half ? 1 : min(TG, nfull - tile0);
            for (int seg = 0; seg < p.nseg; ++seg) {
                for (int j = 0; j < nt_here; ++j) {
                    if (stage >= p.NS) mbar_wait(empty0 + slot * 8, parity ^ 1u, abort_flag, 2, stage);
                    if (lane == 0) {
                        const int row0 = r0 + (tile0 + j) * tile_rows;
                        const uint32_t fullb = full0 + slot * 8;
                        const uint32_t sbase = ring_u32 + (uint32_t)slot * (uint32_t)p.stage_bytes;
                        mbar_expect_tx(fullb, (uint32_t)(half ? 8 : 16) * (uint32_t)(p.RS + p.AS));
                        if constexpr (split_gu) {
                            // rows 0..7 of the tile: gate rows row0.., rows 8..15: the up rows of the same outputs
                            tma_load_2d(sbase, &p.wmap8, seg * p.SB * 4, row0, fullb);
                            tma_load_2d(sbase + 8 * p.RS, &p.wmap8, seg * p.SB * 4, n_own + row0, fullb);
                            tma_load_2d(sbase + 16 * p.RS, &p.amap8, seg * p.SB, row0, fullb);
                            tma_load_2d(sbase + 16 * p.RS + 8 * p.AS, &p.amap8, seg * p.SB, n_own + row0, fullb);
                        } else {
                            tma_load_2d(sbase, half ? &p.wmap8 : &p.wmap16, seg * p.SB * 4, row0, fullb);
                            tma_load_2d(sbase + 16 * p.RS, half ? &p.amap8 : &p.amap16, seg * p.SB, row0, fullb);
                        }
                    }
                    __syncwarp();
                    ++stage;
                    if (++slot == p.NS) { slot = 0; parity ^= 1u; }
                }
            }
            tile0 += nt_here;
        }
        if (p.pf_packed) {
            // every load of this launch is in flight: pull the head of this CTA's share of the next
            // launch's weights into L2 (first SG_PF_ROWS rows, up to SG_PF_ROW_BYTES of each)
            const int f0 = (bid * p.pf_h_base + min(bid, p.pf_h_rem)) * 8;
            const int f1 = min(f0 + (p.pf_h_base + (bid < p.pf_h_rem ? 1 : 0)) * 8, p.pf_N);
            const uint32_t wb = (uint32_t)min(p.pf_row_bytes, SG_PF_ROW_BYTES);
            const uint32_t ab = (uint32_t)min(p.pf_am_row_bytes, SG_PF_ROW_BYTES / 8) & ~15u;
            for (int row = f0 + lane; row < min(f1, f0 + SG_PF_ROWS); row += 32) {
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.pf_packed + (int64_t)row * p.pf_row_bytes), "r"(wb) : "memory");
                if (ab) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<const uint8_t*>(p.pf_absmax) + (int64_t)row * p.pf_am_row_bytes), "r"(ab) : "memory");
            }
        }
        return;
    }

    // ----------------------------------- compute warps ------------------------------------------
    if (p.x_staged && warp == 0) {
        // the activations come from the predecessor grid: wait for it here, start the copy, and let the
        // table build below hide its latency
        if (lane == 0) {
            mbar_init(xbar, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        griddep_wait();
        const uint32_t x_row_bytes = (uint32_t)(p.K * 2) * (p.prologue == 2 ? 2u : 1u);
        if (lane == 0) mbar_expect_tx(xbar, (uint32_t)p.M * x_row_bytes);
        __syncwarp();
        if (lane < p.M)
            bulk_g2s(xs_u32 + lane * p.x_stride, static_cast<const uint8_t*>(p.x) + (int64_t)lane * x_row_bytes,
                     x_row_bytes, xbar);
    }
    lut_build<T, CW>(lut_ptr, level, warp, lane);
    float dq_off = 0.0f;
    if (DQ) {
        if (tid < 256) reinterpret_cast<float*>(smem + p.off_c256)[tid] = __ldg(p.code256 + tid);
        dq_off = __ldg(p.offset);
    }
    const uint32_t c256 = s0 + (uint32_t)p.off_c256;
    // barriers armed (producer) and table complete (compute warps) for every compute warp after this
    asm volatile("bar.sync 2, %0;" ::"n"((CW + 1) * 32) : "memory");
    griddep_launch();
    // RMSNorm weights are parameters, not activations: fetch them before waiting for the predecessor
    constexpr int NTH = CW * 32;
    constexpr int NWC = 8;                          // pairs per thread held in registers (K <= 16 * NTH)
    __nv_bfloat162 nw_cache[NWC];
    const bool nw_cached = p.prologue == 1 && p.K / 2 <= NWC * NTH;
    if (nw_cached) {
        const __nv_bfloat162* nw = static_cast<const __nv_bfloat162*>(p.norm_w);
#pragma unroll
        for (int j = 0; j < NWC; ++j) {
            const int i = tid + j * NTH;
            nw_cache[j] = i < p.K / 2 ? nw[i] : __floats2bfloat162_rn(0.0f, 0.0f);
        }
    }
    griddep_wait();
    if (p.x_staged) mbar_wait(xbar, 0u, abort_flag, 3, -1);

    // ---- optional prologue on the staged activations (in place, every CTA for itself) ----------
    if (p.prologue != 0) {
        uint8_t* const xsp = smem + p.off_x;
        const int ctid = tid;                       // 0 .. CW*32-1
        if (p.prologue == 1) {
            float* const red = part;                // 2*CW floats of scratch (free before the first group ends)
            for (int m = 0; m < p.M; ++m) {
                __nv_bfloat162* row = reinterpret_cast<__nv_bfloat162*>(xsp + m * p.x_stride);
                float* const redm = red + (m & 1) * CW;   // alternate so one barrier per row is enough
                if (nw_cached) {
                    float2 v[NWC];
                    float ss = 0.0f;
#pragma unroll
                    for (int j = 0; j < NWC; ++j) {
                        const int i = ctid + j * NTH;
                        v[j] = i < p.K / 2 ? __bfloat1622float2(row[i]) : make_float2(0.0f, 0.0f);
                        ss += v[j].x * v[j].x + v[j].y * v[j].y;
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    if (lane == 0) redm[warp] = ss;
                    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
                    float tot = 0.0f;
#pragma unroll
                    for (int w = 0; w < CW; ++w) tot += redm[w];
                    const float r = rsqrtf(tot / (float)p.K + p.eps);
#pragma unroll
                    for (int j = 0; j < NWC; ++j) {
                        const int i = ctid + j * NTH;
                        const float2 gw = __bfloat1622float2(nw_cache[j]);
                        if (i < p.K / 2) row[i] = __floats2bfloat162_rn(v[j].x * r * gw.x, v[j].y * r * gw.y);
                    }
                } else {
                    float ss = 0.0f;
                    for (int i = ctid; i < p.K / 2; i += NTH) {
                        const float2 v = __bfloat1622float2(row[i]);
                        ss += v.x * v.x + v.y * v.y;
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    if (lane == 0) redm[warp] = ss;
                    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
                    float tot = 0.0f;
#pragma unroll
                    for (int w = 0; w < CW; ++w) tot += redm[w];
                    const float r = rsqrtf(tot / (float)p.K + p.eps);
                    const __nv_bfloat162* nw = static_cast<const __nv_bfloat162*>(p.norm_w);
                    for (int i = ctid; i < p.K / 2; i += NTH) {
                        const float2 v = __bfloat1622float2(row[i]);
                        const float2 gw = __bfloat1622float2(nw[i]);
                        row[i] = __floats2bfloat162_rn(v.x * r * gw.x, v.y * r * gw.y);
                    }
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
        } else {
            for (int m = 0; m < p.M; ++m) {
                __nv_bfloat162* row = reinterpret_cast<__nv_bfloat162*>(xsp + m * p.x_stride);
                for (int i = ctid; i < p.K / 2; i += NTH) {
                    const float2 gt = __bfloat1622float2(row[i]);
                    const float2 up = __bfloat1622float2(row[i + p.K / 2]);
                    row[i] = __floats2bfloat162_rn(gt.x / (1.0f + __expf(-gt.x)) * up.x, gt.y / (1.0f + __expf(-gt.y)) * up.y);
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
        }
    }

    const uint32_t window_lane = lut_base | (uint32_t)(lane << 2);
    // Warp w owns the adjacent blocks [w * BPW, (w + 1) * BPW) of every stage.  A warp beyond the stage's width
    // (SB < 32; SB is a multiple of 4, so a warp owns all of its blocks or none) reads the stage's last BPW
    // blocks against all-zero activation fragments, so every warp always computes BPW blocks.
    const bool live_warp = warp * BPW < p.SB;
    const int b0 = min(warp * BPW, p.SB - BPW);
    uint32_t a_off[BPW];
#pragma unroll
    for (int bi = 0; bi < BPW; ++bi) a_off[bi] = (uint32_t)(g * p.RS + (b0 + bi) * 32 + q * 8);
    const uint32_t am_off = (uint32_t)(16 * p.RS + g * p.AS + b0 * (DQ ? 1 : 4));
    const uint32_t rs8 = 8u * (uint32_t)p.RS, as8 = 8u * (uint32_t)p.AS;
    const uint32_t stage_bytes = (uint32_t)p.stage_bytes;
    const int NS = p.NS;
    const int Mc = p.M;

    float acc[TG][NT][4];
    int stage = 0;
    uint32_t slot = 0, parity = 0;

    // activation fragments of this warp's blocks in segment `seg`: 16 consecutive values of
    // activation row m = g (+8) per block
    auto load_xf = [&](uint32_t (&xf)[BPW][NT][8], int seg) {
#pragma unroll
        for (int bi = 0; bi < BPW; ++bi) {
            const int kb = seg * p.SB + b0 + bi;
            const bool live = live_warp;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int m = g + nt * 8;
                uint4 v0 = make_uint4(0u, 0u, 0u, 0u), v1 = v0;
                if (live && m < Mc) {
                    if (p.x_staged) {
                        const uint32_t src = xs_u32 + (uint32_t)(m * p.x_stride + ((kb * 64 + q * 16) << 1));
                        v0 = lds128(src);
                        v1 = lds128(src + 16);
                    } else {
                        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.x) +
                                                                          (((int64_t)m * p.K + kb * 64 + q * 16) << 1));
                        v0 = __ldg(src);
                        v1 = __ldg(src + 1);
                    }
                }
                xf[bi][nt][0] = v0.x; xf[bi][nt][1] = v0.y; xf[bi][nt][2] = v0.z; xf[bi][nt][3] = v0.w;
                xf[bi][nt][4] = v1.x; xf[bi][nt][5] = v1.y; xf[bi][nt][6] = v1.z; xf[bi][nt][7] = v1.w;
            }
        }
    };

    // one stage: wait for the box, compute, hand the slot back
    // DQ: second-level scales of this lane's rows (g, g+8 of the tile starting at row0_) in segment seg_: one
    // scale per 256 consecutive first-level blocks of the flattened weight; SB (16 or 32) divides K/64, so the
    // SB blocks of a row's segment start at a multiple of SB and never straddle a multiple of 256
    auto load_scales = [&](float (&sc)[2], int row0_, int seg_) {
        if (DQ) {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int row = min(split_gu ? row0_ + g + hh * n_own : row0_ + g + 8 * hh, p.N - 1);
                sc[hh] = __ldg(p.scale2 + (((int64_t)row * p.KB + seg_ * p.SB) >> 8));
            }
        }
    };
#define NF4_DO_STAGE(HALF_, XF_, ACC_, ROW0_, SEG_)                                                                 \
    do {                                                                                                           \
        float sc_[2];                                                                                              \
        load_scales(sc_, ROW0_, SEG_);                                                                             \
        mbar_wait(full0 + slot * 8, parity, abort_flag, 1, stage);                                                  \
        stage_compute<T, NT, BPW, HALF_, DQ>(ring_u32 + slot * stage_bytes, a_off, am_off, rs8, as8, window_lane, XF_, ACC_, sc_, c256, dq_off); \
        __syncwarp();                                                                                              \
        if (lane == 0) mbar_arrive(empty0 + slot * 8);                                                              \
        ++stage;                                                                                                   \
        if (++slot == (uint32_t)NS) { slot = 0; parity ^= 1u; }                                                     \
    } while (0)

    // end of a group: the CW partial sums of every output meet in shared memory (fixed order)
    auto finish_group = [&](int tile0, int nt_here) {
        float* const mine = part + warp * (TG * Mc * 16);   // layout part[warp][j][m][16 rows]
#pragma unroll
        for (int j = 0; j < TG; ++j) {
            if (j < nt_here) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int m = nt * 8 + 2 * q;
                    if (m < Mc) {
                        mine[(j * Mc + m) * 16 + g] = acc[j][nt][0];
                        mine[(j * Mc + m) * 16 + g + 8] = acc[j][nt][2];
                    }
                    if (m + 1 < Mc) {
                        mine[(j * Mc + m + 1) * 16 + g] = acc[j][nt][1];
                        mine[(j * Mc + m + 1) * 16 + g + 8] = acc[j][nt][3];
                    }
                }
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
        if (p.epilogue == 1) {
            // SwiGLU: weight rows 2i / 2i+1 are gate_i / up_i; both sums are rounded to the activation
            // type first (what a separate kernel would read back), then h_i = silu(gate_i) * up_i
            const int pairs = nt_here * Mc * 8;
            const int half_n = p.N >> 1;
            for (int o = tid; o < pairs; o += CW * 32) {
                const int pr = o & 7;
                const int jm = o >> 3;
                const int j = jm / Mc;
                const int m = jm - j * Mc;
                const int grow = r0 + (tile0 + j) * 16 + 2 * pr;
                if (grow < r1) {
                    float sg = 0.0f, su = 0.0f;
                    const int idx = jm * 16 + 2 * pr;
#pragma unroll
                    for (int w = 0; w < CW; ++w) {
                        sg += part[w * (TG * Mc * 16) + idx];
                        su += part[w * (TG * Mc * 16) + idx + 1];
                    }
                    const float gt = Elem<T>::to_f32(Elem<T>::from_f32(sg));
                    const float up = Elem<T>::to_f32(Elem<T>::from_f32(su));
                    static_cast<T*>(p.y)[(int64_t)m * half_n + (grow >> 1)] = Elem<T>::from_f32(gt / (1.0f + __expf(-gt)) * up);
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
            return;
        }
        if constexpr (GU) {
            // SwiGLU over split halves: rows 0..7 of a tile are gate_i, rows 8..15 the up_i of the same outputs
            const int pairs = nt_here * Mc * 8;
            for (int o = tid; o < pairs; o += CW * 32) {
                const int pr = o & 7;
                const int jm = o >> 3;
                const int j = jm / Mc;
                const int m = jm - j * Mc;
                const int grow = r0 + (tile0 + j) * 8 + pr;
                if (grow < r1) {
                    float sg = 0.0f, su = 0.0f;
                    const int idx = jm * 16 + pr;
#pragma unroll
                    for (int w = 0; w < CW; ++w) {
                        sg += part[w * (TG * Mc * 16) + idx];
                        su += part[w * (TG * Mc * 16) + idx + 8];
                    }
                    const float gt = Elem<T>::to_f32(Elem<T>::from_f32(sg));
                    const float up = Elem<T>::to_f32(Elem<T>::from_f32(su));
                    static_cast<T*>(p.y)[(int64_t)m * n_own + grow] = Elem<T>::from_f32(gt / (1.0f + __expf(-gt)) * up);
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
            return;
        }
        const int outputs = nt_here * Mc * 16;
        for (int o = tid; o < outputs; o += CW * 32) {
            const int row = o & 15;
            const int jm = o >> 4;           // j * Mc + m
            const int j = jm / Mc;
            const int m = jm - j * Mc;
            const int grow = r0 + (tile0 + j) * 16 + row;
            if (grow < r1) {
                float sum = 0.0f;
#pragma unroll
                for (int w = 0; w < CW; ++w) sum += part[w * (TG * Mc * 16) + o];
                if (p.bias) sum += Elem<T>::to_f32(static_cast<const T*>(p.bias)[grow]);
                if (p.residual) sum += Elem<T>::to_f32(static_cast<const T*>(p.residual)[(int64_t)m * p.N + grow]);
                static_cast<T*>(p.y)[(int64_t)m * p.N + grow] = Elem<T>::from_f32(sum);
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    };

    auto zero_acc = [&]() {
#pragma unroll
        for (int j = 0; j < TG; ++j)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[j][nt][e] = 0.0f;
    };

    int tile0 = 0;
    // complete groups of TG full tiles: no per-stage conditionals
    for (; tile0 + TG <= nfull; tile0 += TG) {
        zero_acc();
        for (int seg = 0; seg < p.nseg; ++seg) {
            uint32_t xf[BPW][NT][8];
            load_xf(xf, seg);
#pragma unroll
            for (int j = 0; j < TG; ++j) NF4_DO_STAGE(false, xf, acc[j], r0 + (tile0 + j) * tile_rows, seg);
        }
        finish_group(tile0, TG);
    }
    // the remaining full tiles
    if (tile0 < nfull) {
        const int nt_here = nfull - tile0;
        zero_acc();
        for (int seg = 0; seg < p.nseg; ++seg) {
            uint32_t xf[BPW][NT][8];
            load_xf(xf, seg);
#pragma unroll
            for (int j = 0; j < TG; ++j)
                if (j < nt_here) NF4_DO_STAGE(false, xf, acc[j], r0 + (tile0 + j) * tile_rows, seg);
        }
        finish_group(tile0, nt_here);
        tile0 = nfull;
    }
    // the half tile
    if (tile0 < ntiles) {
        zero_acc();
        for (int seg = 0; seg < p.nseg; ++seg) {
            uint32_t xf[BPW][NT][8];
            load_xf(xf, seg);
            NF4_DO_STAGE(true, xf, acc[0], r0 + tile0 * 16, seg);
        }
        finish_group(tile0, 1);
    }
#undef NF4_DO_STAGE
}

// ---------------------------------------------------------------------------------------------

static thread_local bool g_launch_pdl = false;   // set by the entry point for the duration of one call

template <typename T, int NT, int TG, int CW, bool DQ, bool GU>
static int launch_staged_as(const StagedParams& p, int grid, cudaStream_t stream) {
    static bool configured[64] = {false};
    int dev = 0;
    NF4_CUDA_TRY(cudaGetDevice(&dev));
    NF4_REQUIRE(dev < 64, NF4_ERR_LIMIT, "gemv: device ordinal %d (at most 64 devices per process)", dev);
    if (!configured[dev]) {
        NF4_CUDA_TRY(cudaFuncSetAttribute(gemv_staged_kernel<T, NT, TG, CW, DQ, GU>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMV_SMEM));
        configured[dev] = true;
    }
    if (g_launch_pdl) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)grid);
        cfg.blockDim = dim3((CW + 1) * 32);
        cfg.dynamicSmemBytes = GEMV_SMEM;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        NF4_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_staged_kernel<T, NT, TG, CW, DQ, GU>, p));
    } else {
        gemv_staged_kernel<T, NT, TG, CW, DQ, GU><<<grid, (CW + 1) * 32, GEMV_SMEM, stream>>>(p);
    }
    NF4_CUDA_TRY(cudaGetLastError());
    return NF4_OK;
}

// the double-quantized form and the SwiGLU-over-halves epilogue exist for bf16 only (the type of every
// configuration that uses them), and not combined
template <typename T, int NT, int TG, int CW>
static int launch_staged(const StagedParams& p, int grid, cudaStream_t stream) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        if (p.absmax_u8 && p.epilogue != 2) return launch_staged_as<T, NT, TG, CW, true, false>(p, grid, stream);
        if (p.epilogue == 2 && !p.absmax_u8) return launch_staged_as<T, NT, TG, CW, false, true>(p, grid, stream);
    }
    if (p.epilogue == 2) return -2;
    return launch_staged_as<T, NT, TG, CW, false, false>(p, grid, stream);
}

// ---- tensor maps ----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

struct MapSet { CUtensorMap w16, w8, a16, a8; };

// One set of maps per (weight pointer, absmax pointer, N, K, SB); a map encodes only address and
// geometry, so it stays valid when the buffer's contents change.
static int get_maps(const uint8_t* packed, const void* absmax, bool dq, int N, int K, int SB, MapSet* out) {
    typedef std::tuple<const void*, const void*, int, int, int, int> Key;
    static std::map<Key, MapSet> cache;
    static std::mutex mu;
    int dev = 0;
    NF4_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    const Key key(packed, absmax, N, K, dq ? -SB : SB, dev);
    auto it = cache.find(key);
    if (it == cache.end()) {
        EncodeTiledFn enc = encode_fn();
        NF4_REQUIRE(enc, NF4_ERR_CUDA, "gemv: cuTensorMapEncodeTiled is not available from this driver");
        if (cache.size() > 4096) cache.clear();
        MapSet ms;
        const int KB = K / 64;
        const cuuint32_t estr[2] = {1, 1};
        for (int i = 0; i < 2; ++i) {
            const cuuint32_t rows = i == 0 ? 16 : 8;
            const cuuint64_t wdim[2] = {(cuuint64_t)(K / 16), (cuuint64_t)N};      // uint64 elements per row
            const cuuint64_t wstr[1] = {(cuuint64_t)(K / 2)};
            const cuuint32_t wbox[2] = {(cuuint32_t)(SB * 4 + 4), rows};
            CUresult r = enc(i == 0 ? &ms.w16 : &ms.w8, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t*>(packed), wdim, wstr,
                             wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            NF4_REQUIRE(r == CUDA_SUCCESS, NF4_ERR_CUDA, "gemv: cuTensorMapEncodeTiled(weights) failed with %d", (int)r);
            // absmax: fp32 [N][KB] in boxes of SB + 4 values, or (double quantization) uint8 [N][KB] in boxes of SB + 16
            const cuuint64_t adim[2] = {(cuuint64_t)KB, (cuuint64_t)N};
            const cuuint64_t astr[1] = {(cuuint64_t)KB * (dq ? 1 : 4)};
            const cuuint32_t abox[2] = {(cuuint32_t)(dq ? SB + 16 : SB + 4), rows};
            r = enc(i == 0 ? &ms.a16 : &ms.a8, dq ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                    const_cast<void*>(absmax), adim, astr, abox,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            NF4_REQUIRE(r == CUDA_SUCCESS, NF4_ERR_CUDA, "gemv: cuTensorMapEncodeTiled(absmax) failed with %d", (int)r);
        }
        it = cache.emplace(key, ms).first;
    }
    *out = it->second;      // copied while the lock is held: another thread may clear the cache
    return NF4_OK;
}

// Returns NF4_OK after launching, an error code, or -1 when the shape does not fit this kernel (the
// caller then takes the direct-load kernel).
template <typename T>
int gemv_staged_try(const void* x, int M, int K, const uint8_t* packed, const float* absmax, const float* code16, int N,
                    const void* bias, const void* residual, void* y, cudaStream_t stream, const GemvOptions& opt) {
    const int KB = K / 64;
    if (KB % 4 != 0) return -1;
    const bool dq = opt.dq_absmax_u8 != nullptr;
    const void* am_ptr = dq ? static_cast<const void*>(opt.dq_absmax_u8) : static_cast<const void*>(absmax);
    if (reinterpret_cast<uintptr_t>(packed) % 16 || reinterpret_cast<uintptr_t>(am_ptr) % 16 ||
        reinterpret_cast<uintptr_t>(x) % 16)
        return -1;
    int SB = 0;
    if (dq) {
        // uint8 absmax rows: the row pitch (KB bytes) and the box width (SB + 16 bytes) must be multiples of 16
        if (!std::is_same<T, __nv_bfloat16>::value || KB % 16 != 0) return -1;
        SB = KB % 32 == 0 ? 32 : 16;
    } else {
        for (int c = 32; c >= 8; c -= 4)
            if (KB % c == 0) { SB = c; break; }
    }
    if (SB == 0) return -1;
    if (const char* env = getenv("NF4_GEMV_SB")) {   // tuning override: blocks per stage
        const int v = atoi(env);
        if (v >= 8 && v <= 32 && v % 4 == 0 && KB % v == 0 && !dq) SB = v;
    }
    const int NT = M <= 8 ? 1 : 2;
    const int sms = sm_count();
    if (opt.epilogue == 2 && (N % 16 != 0)) return -2;
    const int H = opt.epilogue == 2 ? N / 16 : (N + 7) / 8;      // halves of 8 rows (epilogue 2: of 8 gate rows)
    int grid = sms;
    if (opt.epilogue == 2) {
        if (grid > H) grid = H;
    } else if (grid > (H + 1) / 2) {
        grid = (H + 1) / 2;
    }
    const int tiles = opt.epilogue == 2 ? (H + grid - 1) / grid : ((H + grid - 1) / grid + 1) / 2;
    // 16 compute warps; 8 for two column tiles whose activations stay in global memory (more than fit
    // below the table): every group of tiles re-reads the activations from L2, so the groups are made
    // 4 tiles tall, which needs the registers of the 8-warp shape
    int CW = 16;
    if (NT == 2 && (int64_t)M * K * 2 > 40 * 1024) CW = 8;
    if (const char* env = getenv("NF4_GEMV_CW")) {
        const int v = atoi(env);
        if (v == 8 || v == 16) CW = v;
    }
    int TG = (NT == 1 || CW == 8) ? 4 : 2;
    while (TG > 1 && TG / 2 >= tiles) TG /= 2;
    if (const char* env = getenv("NF4_GEMV_TG")) {
        const int v = atoi(env);
        if (v == 1 || v == 2 || (v == 4 && (NT == 1 || CW == 8))) TG = v;
    }

    StagedParams p;
    p.x = x; p.packed = packed; p.absmax = absmax; p.code16 = code16; p.bias = bias; p.residual = residual; p.y = y;
    p.absmax_u8 = opt.dq_absmax_u8; p.scale2 = opt.dq_scale2; p.offset = opt.dq_offset; p.code256 = opt.dq_code256;
    p.M = M; p.N = N; p.K = K; p.KB = KB; p.SB = SB; p.nseg = KB / SB;
    p.h_base = H / grid;
    p.h_rem = H % grid;
    p.pf_packed = nullptr; p.pf_absmax = nullptr; p.pf_N = 0; p.pf_row_bytes = 0; p.pf_am_row_bytes = 0; p.pf_h_base = 0; p.pf_h_rem = 0;
    if (opt.next_packed && opt.next_absmax && opt.next_N > 0 && opt.next_K >= 64 && opt.next_K % 64 == 0 &&
        reinterpret_cast<uintptr_t>(opt.next_packed) % 16 == 0 && reinterpret_cast<uintptr_t>(opt.next_absmax) % 16 == 0 &&
        (opt.next_K / 64) % 4 == 0) {
        // the next launch deals its rows out the same way over (up to) the same number of CTAs
        const int Hn = (opt.next_N + 7) / 8;
        int gn = sms;
        if (gn > (Hn + 1) / 2) gn = (Hn + 1) / 2;
        if (gn == grid) {
            p.pf_packed = opt.next_packed; p.pf_absmax = opt.next_absmax; p.pf_N = opt.next_N;
            p.pf_row_bytes = opt.next_K / 2; p.pf_am_row_bytes = opt.next_K / 64 * 4;
            p.pf_h_base = Hn / gn; p.pf_h_rem = Hn % gn;
        }
    }
    p.RS = SB * 32 + 32;
    p.AS = dq ? SB + 16 : SB * 4 + 16;
    p.stage_bytes = 16 * p.RS + 16 * p.AS;
    p.prologue = opt.prologue; p.norm_w = opt.norm_w; p.eps = opt.eps; p.epilogue = opt.epilogue;
    if (opt.epilogue == 1 && (N % 2 != 0)) return -2;
    p.x_stride = (opt.prologue == 2 ? 4 : 2) * K + 16;
    // Shared-memory map.  The dynamic region starts ~1 KB into the shared window, the table takes
    // the 64 KB aligned window [64K, 128K); below it: barriers, partial sums, staged activations;
    // above it: the ring (every stage and both boxes inside it start on a 128-byte boundary).
    const int low_cap = LUT_WINDOW - 2048;           // leaves room for the window's start offset
    p.off_bars = 0;
    p.off_c256 = 256;
    p.off_part = dq ? 256 + 1024 : 256;
    const int part_bytes = CW * TG * M * 16 * 4;
    p.off_x = (p.off_part + part_bytes + 127) & ~127;
    if (p.off_x > low_cap) return -1;
    p.x_staged = ((int64_t)p.off_x + (int64_t)M * p.x_stride <= low_cap) ? 1 : 0;
    if (opt.prologue != 0 && !p.x_staged) return -2;   // a prologue needs the activations in shared memory
    const int ring_cap = GEMV_SMEM - 2 * LUT_WINDOW;   // the window ends at most 128 KB into the region
    int NS = ring_cap / p.stage_bytes;
    if (NS > SG_MAX_STAGES) NS = SG_MAX_STAGES;
    if (NS < 2) return -1;
    if (const char* env = getenv("NF4_GEMV_NS")) {   // tuning override: ring depth
        const int v = atoi(env);
        if (v >= 2 && v <= NS) NS = v;
    }
    p.NS = NS;
    if (opt.dry_run) return NF4_OK;
    MapSet ms;
    if (int rc = get_maps(packed, am_ptr, dq, N, K, SB, &ms)) return rc;
    p.wmap16 = ms.w16; p.wmap8 = ms.w8; p.amap16 = ms.a16; p.amap8 = ms.a8;

    g_launch_pdl = opt.pdl;
#define NF4_SG(NT_, TG_)                                                        \
    do {                                                                        \
        if (CW == 8) return launch_staged<T, NT_, TG_, 8>(p, grid, stream);     \
        return launch_staged<T, NT_, TG_, 16>(p, grid, stream);                 \
    } while (0)
    if (NT == 1) {
        if (TG == 4) NF4_SG(1, 4);
        if (TG == 2) NF4_SG(1, 2);
        NF4_SG(1, 1);
    } else {
        if (TG == 4) return launch_staged<T, 2, 4, 8>(p, grid, stream);
        if (TG == 2) NF4_SG(2, 2);
        NF4_SG(2, 1);
    }
#undef NF4_SG
}

template int gemv_staged_try<__nv_bfloat16>(const void*, int, int, const uint8_t*, const float*, const float*, int,
                                            const void*, const void*, void*, cudaStream_t, const GemvOptions&);
template int gemv_staged_try<__half>(const void*, int, int, const uint8_t*, const float*, const float*, int, const void*,
                                     const void*, void*, cudaStream_t, const GemvOptions&);

}  // namespace nf4

using namespace nf4;

namespace nf4 {
int gemm_read_error(unsigned int* out4);
int attn_read_error(unsigned int* out4);
int ar_read_error(unsigned int* out4);
int gemm_clear_error();
int attn_clear_error();
int ar_clear_error();
}

extern "C" int nf4_b200_gemv_decode_fits(int64_t M, int64_t N, int64_t K, int prologue) {
    if (M < 1 || M > 16 || N < 1 || K < 64 || K % 64 != 0 || prologue < 0 || prologue > 2) return 0;
    GemvOptions opt;
    opt.prologue = prologue;
    opt.dry_run = true;
    const void* aligned = reinterpret_cast<const void*>(uintptr_t(256));
    return gemv_staged_try<__nv_bfloat16>(aligned, (int)M, (int)K, static_cast<const uint8_t*>(aligned),
                                          static_cast<const float*>(aligned), nullptr, (int)N, nullptr, nullptr, nullptr,
                                          nullptr, opt) == NF4_OK ? 1 : 0;
}

extern "C" int nf4_b200_device_error(unsigned int* host_out4) {
    NF4_REQUIRE(host_out4, NF4_ERR_ARG, "device_error: null pointer");
    NF4_CUDA_TRY(cudaMemcpyFromSymbol(host_out4, g_gemv_error, sizeof(unsigned int) * 4));
    if (host_out4[0] == 0) {   // no GEMV error: report the GEMM kernel's word
        unsigned int g[4] = {0, 0, 0, 0};
        if (int rc = gemm_read_error(g)) return rc;
        for (int i = 0; i < 4; ++i) host_out4[i] = g[i];
    }
    if (host_out4[0] == 0) {   // nor a GEMM error: the attention kernels' word
        unsigned int g[4] = {0, 0, 0, 0};
        if (int rc = attn_read_error(g)) return rc;
        for (int i = 0; i < 4; ++i) host_out4[i] = g[i];
    }
    if (host_out4[0] == 0) {   // ... and the tensor-parallel all-reduce's
        unsigned int g[4] = {0, 0, 0, 0};
        if (int rc = ar_read_error(g)) return rc;
        for (int i = 0; i < 4; ++i) host_out4[i] = g[i];
    }
    return NF4_OK;
}

extern "C" int nf4_b200_device_error_clear(void) {
    const unsigned int zero[4] = {0u, 0u, 0u, 0u};
    NF4_CUDA_TRY(cudaMemcpyToSymbol(g_gemv_error, zero, sizeof(zero)));
    if (int rc = gemm_clear_error()) return rc;
    if (int rc = attn_clear_error()) return rc;
    return ar_clear_error();
}
