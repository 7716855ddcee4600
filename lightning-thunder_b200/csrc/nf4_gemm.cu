// NF4 dequant-GEMM on the 5th-generation tensor cores (tcgen05 / TMEM): prefill, and decode steps of more
// than 8 sequences.
//
//   y[m][n] = sum_k x[m][k] * W[n][k] + bias[n],   W[n][k] = bf16( bf16(code[idx]) * absmax[n][k/64] )
//
// One CTA computes a tile of 128 weight rows x TM (<= 256) activation rows over a range of K blocks.
// Weights are the A operand (UMMA M = 128) and live in TENSOR MEMORY: the dequant warps write bf16 pairs
// straight into TMEM columns (tcgen05.st), so the dequantised matrix never crosses shared memory, whose
// bandwidth the activation operand already uses.  Activations are the B operand (UMMA N = TM), K-major
// bf16 in shared memory with the 128-byte swizzle.  The fp32 accumulator takes TMEM columns [0, TM), the
// 4 weight stages 32 columns each after it.  Per 64-element K block (one quantization block per row):
//   warp 10  (weights)   TMA: packed weights as boxes of 128 rows x 128 bytes (4 K blocks; SWIZZLE_128B so that
//                        16-byte reads of 8 consecutive rows are conflict-free) into a 3-deep ring of their
//                        own -> mbarrier `w_full`: up to 12 K blocks ahead of the dequant warps, however
//                        far the activation ring has got
//   warp 0   (activations) TMA: one box of TM x 64 (SWIZZLE_128B) per K block into a 4-deep ring -> `full`
//   warps 2-9 (dequant)  two threads per weight row, 16 bytes -> 32 bf16 each, through the byte->(bf16,bf16)
//                        table, scaled by the row's fp32 absmax in fp32, rounded once, written to the
//                        thread's TMEM lane (16 columns); tcgen05.wait::st + arrive on `a_ready`; after
//                        the 4th block of a packed stage, arrive on `w_empty`
//   warp 1   (MMA)       one elected thread issues 4 x tcgen05.mma (K = 16 each, A from TMEM) per block and
//                        commits to `empty` (frees both stages) -- after the last block to `acc_done`
// Epilogue (warps 2-5): tcgen05.ld 32 lanes x 16 columns at a time, + bias (+ residual), bf16, store to
// y[m][n] (a warp writes 32 consecutive n for one m: 64-byte segments); or SwiGLU over adjacent lanes.
// Split K (few weight tiles): CTAs of one tile park fp32 partial sums in a workspace, bump an arrival
// counter, and the last one adds the partials in range order (deterministic) and runs the epilogue.
//
// Every mbarrier wait is bounded; a time-out sets a status word (nf4_b200_device_error code 5..9),
// the CTA stops waiting and runs to its end (TMEM is always released).
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>

#include "nf4_common.cuh"

namespace nf4 {

bool gemv_supported(int64_t M, int64_t K, int64_t N, int blocksize, int dtype, const void* x, const void* packed,
                    const void* absmax);
__device__ unsigned int g_gemm_error[4];   // [0] first error code, [1] block, [2] K block, [3] count

// host side: copies the GEMM status word (synchronises)
int gemm_read_error(unsigned int* out4) {
    NF4_CUDA_TRY(cudaMemcpyFromSymbol(out4, g_gemm_error, sizeof(unsigned int) * 4));
    return NF4_OK;
}

constexpr int GM_DQ_WARPS = 8;           // dequant warps: two threads per weight row (half a block each)
constexpr int GM_THREADS = (3 + GM_DQ_WARPS) * 32;   // activation producer, MMA, dequant (the first 4 also run the epilogue), weight producer
constexpr int GM_WPRODUCER = 2 + GM_DQ_WARPS;        // warp index of the weight producer
constexpr int GM_BM = 128;               // weight rows per CTA (UMMA M)
constexpr int GM_STAGES = 4;
constexpr int GM_A_COLS = 32;            // TMEM columns of one weight stage: 64 bf16 per row, two per column
constexpr int GM_WSTAGES = 3;            // packed-weight stages, each GM_WKB K blocks deep
constexpr int GM_WKB = 4;                // K blocks per packed-weight stage: 4 x 32 B = one 128-byte swizzle row
constexpr int GM_PK_BYTES = GM_BM * 128; // one packed-weight stage
constexpr int GM_LUT_BYTES = 256 * 128;  // byte -> (bf16,bf16), one copy per lane
constexpr int GM_MIN_SMEM = 80 * 1024;   // request at least this much: at most two CTAs (2 x 256 TMEM columns) per SM
constexpr int GM_MAX_CTAS_SPLIT = 296;   // split K until about two CTAs per SM exist
constexpr unsigned long long GM_WAIT_LIMIT_NS = 200ull * 1000 * 1000;

struct alignas(64) GemmParams {
    CUtensorMap wmap;     // packed codes uint8 [N][K/2], box 128 B x 128 rows, SWIZZLE_128B
    CUtensorMap xmap;     // activations bf16 [M][K], box 64 x TM, SWIZZLE_128B
    const float* absmax;
    const float* code16;
    const void* bias;
    const void* residual; // bf16 [M][N] added in the epilogue, or null
    void* y;
    float* partials;      // split K: fp32 [group][split][TM][128]
    unsigned* counters;   // split K: one arrival counter per (weight tile, activation tile); zero between launches
    int M, N, K, KB;
    int TM;               // activation rows per CTA: multiple of 16, 32..256
    int tmem_cols;        // power of two >= TM + GM_STAGES * GM_A_COLS
    int splits;           // K is cut into this many ranges, one CTA each
    int epilogue;         // 0: y[m][n];  1: rows are (gate, up) pairs, y[m][n/2] = silu(gate) * up
    int pdl;              // programmatic dependent launch: weights may be fetched before the upstream grid ends
};

__device__ __forceinline__ uint32_t gm_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gm_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void gm_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gm_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool gm_mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long gm_global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void gm_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, int iter) {
    if (gm_mbar_try_wait(bar, parity)) return;
    if (*abort_flag) return;
    const unsigned long long t0 = gm_global_ns();
    while (!gm_mbar_try_wait(bar, parity)) {
        if (*abort_flag) return;
        if (gm_global_ns() - t0 > GM_WAIT_LIMIT_NS) {
            *abort_flag = 1;
            if (atomicCAS(&g_gemm_error[0], 0u, (unsigned)code) == 0u) {
                g_gemm_error[1] = blockIdx.x + blockIdx.y * gridDim.x;
                g_gemm_error[2] = (unsigned)iter;
            }
            atomicAdd(&g_gemm_error[3], 1u);
            return;
        }
    }
}
__device__ __forceinline__ void gm_tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}

// 32 lanes x 16 columns of fp32 from tensor memory into 16 registers per thread
__device__ __forceinline__ void gm_tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t gm_smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3ffffu) >> 4);          // start address
    d |= (uint64_t)1 << 16;                           // leading-dimension byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                 // stride-dimension byte offset: 8 rows x 128 B
    d |= (uint64_t)1 << 46;                           // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                           // SWIZZLE_128B
    return d;
}

// Instruction descriptor: D = f32, A = B = bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t gm_instr_desc(int n) {
    uint32_t d = 0;
    d |= 1u << 4;                      // D format f32
    d |= 1u << 7;                      // A format bf16
    d |= 1u << 10;                     // B format bf16
    d |= (uint32_t)(n >> 3) << 17;     // N >> 3
    d |= (uint32_t)(GM_BM >> 4) << 24; // M >> 4
    return d;
}

__global__ void __launch_bounds__(GM_THREADS, 1) gemm_tcgen05_kernel(const __grid_constant__ GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int TM = p.TM;
    const int b_bytes = TM * 128;

    // shared-memory map (all stage bases 1024-byte aligned)
    uint8_t* const b_base = smem;                                      // GM_STAGES x TM*128
    uint8_t* const pk_base = b_base + GM_STAGES * b_bytes;             // GM_WSTAGES x 16 KB
    uint8_t* const lut = pk_base + GM_WSTAGES * GM_PK_BYTES;           // 32 KB
    uint64_t* const bars = reinterpret_cast<uint64_t*>(lut + GM_LUT_BYTES);
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
    volatile int* const abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* const last_flag = abort_flag + 1;
    const uint32_t full0 = gm_smem_u32(bars), aready0 = full0 + 8 * GM_STAGES, empty0 = full0 + 16 * GM_STAGES,
                   accdone = full0 + 24 * GM_STAGES, wfull0 = accdone + 8, wempty0 = wfull0 + 8 * GM_WSTAGES;

    const int n0 = blockIdx.x * GM_BM;
    const int mtile = blockIdx.y / p.splits;
    const int split = blockIdx.y - mtile * p.splits;
    const int m0 = mtile * TM;
    // this CTA's range of 64-element K blocks (never empty: splits <= KB)
    const int kb_begin = (int)((int64_t)p.KB * split / p.splits);
    const int kb_end = (int)((int64_t)p.KB * (split + 1) / p.splits);

    if (tid == 0) {
        for (int s = 0; s < GM_STAGES; ++s) {
            gm_mbar_init(full0 + 8 * s, 1);
            gm_mbar_init(aready0 + 8 * s, GM_DQ_WARPS);   // one arrival per dequant warp
            gm_mbar_init(empty0 + 8 * s, 1);              // tcgen05.commit
        }
        for (int s = 0; s < GM_WSTAGES; ++s) {
            gm_mbar_init(wfull0 + 8 * s, 1);
            gm_mbar_init(wempty0 + 8 * s, GM_DQ_WARPS);   // every dequant warp has read its rows
        }
        gm_mbar_init(accdone, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // TMEM allocation by one full warp; the base address lands in shared memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gm_smem_u32(tmem_slot)), "r"(p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp >= 2 && warp < GM_WPRODUCER) {
        // byte -> (bf16(code[hi]), bf16(code[lo])) table, one copy per lane (conflict-free lookups)
        const float mine = __ldg(p.code16 + (lane & 15));
        for (int e = warp - 2; e < 256; e += GM_DQ_WARPS) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(__shfl_sync(0xffffffffu, mine, e >> 4), __shfl_sync(0xffffffffu, mine, e & 15));
            *reinterpret_cast<uint32_t*>(lut + e * 128 + lane * 4) = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;
    if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ------------------------------ activation producer -----------------------------------
        int slot = 0;
        uint32_t parity = 0;
        if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");   // x comes from the upstream grid
        for (int kb = kb_begin; kb < kb_end; ++kb) {
            gm_wait(empty0 + 8 * slot, parity ^ 1u, abort_flag, 6, kb);
            if (lane == 0) {
                const uint32_t fb = full0 + 8 * slot;
                gm_mbar_expect_tx(fb, (uint32_t)b_bytes);
                gm_tma_2d(gm_smem_u32(b_base + slot * b_bytes), &p.xmap, kb * 64, m0, fb);
            }
            __syncwarp();
            if (++slot == GM_STAGES) { slot = 0; parity ^= 1u; }
        }
    } else if (warp == GM_WPRODUCER) {
        // -------------------------------- weight producer --------------------------------------
        // packed weights: one box of 128 rows x 128 bytes (GM_WKB K blocks) per weight stage, running up to
        // GM_WSTAGES stages ahead of the dequant warps whatever the activation ring does; the weights do
        // not depend on the upstream grid, so nothing here waits for it
        int wslot = 0;
        uint32_t wparity = 0;
        for (int kb = kb_begin; kb < kb_end; kb += GM_WKB) {
            gm_wait(wempty0 + 8 * wslot, wparity ^ 1u, abort_flag, 9, kb);
            if (lane == 0) {
                gm_mbar_expect_tx(wfull0 + 8 * wslot, (uint32_t)GM_PK_BYTES);
                gm_tma_2d(gm_smem_u32(pk_base + wslot * GM_PK_BYTES), &p.wmap, kb * 32, n0, wfull0 + 8 * wslot);
            }
            __syncwarp();
            if (++wslot == GM_WSTAGES) { wslot = 0; wparity ^= 1u; }
        }
    } else if (warp == 1) {
        // ------------------------------------ MMA issuer ---------------------------------------
        const uint32_t idesc = gm_instr_desc(TM);
        int slot = 0;
        uint32_t parity = 0;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
            gm_wait(full0 + 8 * slot, parity, abort_flag, 5, kb);      // activations landed
            gm_wait(aready0 + 8 * slot, parity, abort_flag, 7, kb);    // weights dequantised
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const uint32_t a_tmem = tmem_d + (uint32_t)(TM + slot * GM_A_COLS);
                const uint64_t bdesc = gm_smem_desc(gm_smem_u32(b_base + slot * b_bytes));
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t accumulate = (kb > kb_begin || k > 0) ? 1u : 0u;
                    // 16 K elements per instruction: 8 TMEM columns of the weights, 32 bytes (+2 in the
                    // descriptor's address field) inside the activations' swizzle atom
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "setp.ne.u32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                        ::"r"(tmem_d), "r"(a_tmem + (uint32_t)(8 * k)), "l"(bdesc + (uint64_t)(2 * k)), "r"(idesc), "r"(accumulate)
                        : "memory");
                }
                // frees the stage once these MMAs have read it
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(empty0 + 8 * slot) : "memory");
                if (kb == kb_end - 1)
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(accdone) : "memory");
            }
            __syncwarp();
            if (++slot == GM_STAGES) { slot = 0; parity ^= 1u; }
        }
    } else {
        // ------------------------------------ dequant warps -------------------------------------
        // a warp may touch only the TMEM lane quarter warp % 4, so rows follow that numbering
        const int q = warp & 3;
        const int r = q * 32 + lane;            // weight row inside the tile = TMEM lane
        const int hsel = (warp - 2) >> 2;       // which half of the row's 64-block: bytes [16*hsel, 16*hsel+16)
        const int grow = n0 + r;
        const uint32_t lut_lane = gm_smem_u32(lut) + (uint32_t)lane * 4u;
        const float* const am_row = p.absmax + (int64_t)(grow < p.N ? grow : 0) * p.KB;
        const uint8_t* const pk_row = pk_base + r * 128;
        const int rsw = r & 7;
        int slot = 0;                            // TMEM weight stage (= activation stage) of the current K block
        uint32_t parity = 0;
        int wslot = 0;                           // packed stage the read-ahead is in
        uint32_t wparity = 0;
        int pending = -1;                        // TMEM stage written last, not yet announced
        float am_next = grow < p.N ? __ldg(am_row + kb_begin) : 0.0f;
        // The loop is software-pipelined over K blocks: the packed bytes of block kb+1 are read while block kb
        // is converted, and the tcgen05.st of block kb is only waited for (and announced) after block kb+1
        // has been converted, so neither latency sits on the chain.
        gm_wait(wfull0, 0u, abort_flag, 5, kb_begin);
        uint4 w_next = *reinterpret_cast<const uint4*>(pk_row + ((hsel ^ rsw) << 4));
        for (int kb = kb_begin; kb < kb_end; ++kb) {
            const float am = am_next;
            const uint4 w4 = w_next;
            const int j = (kb - kb_begin) % GM_WKB;                     // K block inside the packed stage
            const int rel_slot = wslot;                                 // packed stage of this K block
            if (kb + 1 < kb_end) {
                am_next = grow < p.N ? __ldg(am_row + kb + 1) : 0.0f;
                int jn = j + 1;
                if (jn == GM_WKB) {
                    jn = 0;
                    if (++wslot == GM_WSTAGES) { wslot = 0; wparity ^= 1u; }
                    gm_wait(wfull0 + 8 * wslot, wparity, abort_flag, 5, kb + 1);   // next packed stage landed
                }
                // 16 bytes of this row: logical 16-byte chunk 2j + hsel of the 128-byte row, at its swizzled place
                w_next = *reinterpret_cast<const uint4*>(pk_row + wslot * GM_PK_BYTES + (((2 * jn + hsel) ^ rsw) << 4));
            }
            const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
            uint32_t pair[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {      // one word = 4 packed bytes = 8 weights; all 16 lookups in flight at once
                const uint32_t byte = __byte_perm(words[i >> 2], 0u, 0x4440 | (i & 3));
                asm("ld.shared.b32 %0, [%1];" : "=r"(pair[i]) : "r"(lut_lane + byte * 128u));
            }
            if (j == GM_WKB - 1 || kb == kb_end - 1) {
                // this warp's last read of the packed stage has been consumed: hand the stage back
                __syncwarp();
                if (lane == 0) gm_mbar_arrive(wempty0 + 8 * rel_slot);
            }
            uint32_t out[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float lo = __uint_as_float(pair[i] << 16) * am;
                const float hi = __uint_as_float(pair[i] & 0xffff0000u) * am;
                const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                out[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
            if (pending >= 0) {
                // the previous block's tcgen05.st has had a whole block's conversion to complete
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) gm_mbar_arrive(aready0 + 8 * pending);
            }
            gm_wait(empty0 + 8 * slot, parity ^ 1u, abort_flag, 6, kb); // the weight stage in TMEM is free
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // 16 columns (32 consecutive K elements) of this thread's lane
            const uint32_t taddr = tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)(TM + slot * GM_A_COLS + hsel * 16);
            asm volatile(
                "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                ::"r"(taddr), "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3]), "r"(out[4]), "r"(out[5]), "r"(out[6]),
                  "r"(out[7]), "r"(out[8]), "r"(out[9]), "r"(out[10]), "r"(out[11]), "r"(out[12]), "r"(out[13]), "r"(out[14]),
                  "r"(out[15]) : "memory");
            pending = slot;
            if (++slot == GM_STAGES) { slot = 0; parity ^= 1u; }
        }
        if (pending >= 0) {
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) gm_mbar_arrive(aready0 + 8 * pending);
        }
        if (warp >= 6) goto done;               // the epilogue needs one warp per TMEM lane quarter
        // ------------------------------------ epilogue ------------------------------------------
        gm_wait(accdone, 0u, abort_flag, 8, kb_end);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int gn = grow;                    // accumulator lane = weight row
        const int mlim = min(TM, p.M - m0);     // activation rows of this tile that exist
        const int group = mtile * gridDim.x + blockIdx.x;
        const uint32_t tacc = tmem_d + ((uint32_t)(q * 32) << 16);
        bool finish = true;
        if (p.splits > 1) {
            // every split parks its fp32 partial sums; the CTA that arrives last adds them in split order
            if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");   // the previous launch may still use the workspace
            float* const mine = p.partials + ((int64_t)(group * p.splits + split) * TM) * 128 + r;
            for (int c0 = 0; c0 < mlim; c0 += 16) {
                uint32_t v[16];
                gm_tmem_ld16(tacc + (uint32_t)c0, v);
#pragma unroll
                for (int j = 0; j < 16; ++j) __stcg(mine + (c0 + j) * 128, __uint_as_float(v[j]));
            }
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (tid == 64) {
                const unsigned prev = atomicAdd(p.counters + group, 1u);
                const int last = prev == (unsigned)(p.splits - 1);
                if (last) p.counters[group] = 0u;       // ready for the next launch
                *last_flag = last;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            finish = *last_flag != 0;
            __threadfence();
        }
        if (finish) {
            if (p.pdl && p.residual && p.splits == 1) asm volatile("griddepcontrol.wait;" ::: "memory");
            const float bias = (p.bias && gn < p.N) ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[gn]) : 0.0f;
            __nv_bfloat16* const y = static_cast<__nv_bfloat16*>(p.y);
            const __nv_bfloat16* const res = static_cast<const __nv_bfloat16*>(p.residual);
            for (int c0 = 0; c0 < mlim; c0 += 16) {
                float v[16];
                if (p.splits > 1) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                    const float* src = p.partials + ((int64_t)(group * p.splits) * TM + c0) * 128 + r;
                    for (int s = 0; s < p.splits; ++s, src += TM * 128) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] += __ldcg(src + j * 128);
                    }
                } else {
                    uint32_t u[16];
                    gm_tmem_ld16(tacc + (uint32_t)c0, u);
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(u[j]);
                }
                if (p.epilogue == 1) {
                    // SwiGLU: lanes 2i / 2i+1 hold gate_i / up_i; both are rounded to bf16 first (what a
                    // separate kernel would read back), then h_i = silu(gate_i) * up_i
                    const int half_n = p.N >> 1;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float mine = __bfloat162float(__float2bfloat16_rn(v[j] + bias));
                        const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
                        const int m = m0 + c0 + j;
                        if (!(lane & 1) && gn + 1 < p.N && m < p.M)
                            y[(int64_t)m * half_n + (gn >> 1)] = __float2bfloat16_rn(mine / (1.0f + __expf(-mine)) * other);
                    }
                } else if (gn < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = m0 + c0 + j;
                        if (m < p.M) {
                            float o = v[j] + bias;
                            if (res) o += __bfloat162float(res[(int64_t)m * p.N + gn]);
                            y[(int64_t)m * p.N + gn] = __float2bfloat16_rn(o);
                        }
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
done:
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(p.tmem_cols) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------

typedef CUresult (*GmEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static GmEncodeFn gm_encode_fn() {
    static GmEncodeFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<GmEncodeFn>(ptr);
    }
    return fn;
}

static int gemm_smem_bytes(int TM) {
    const int need = GM_STAGES * TM * 128 + GM_WSTAGES * GM_PK_BYTES + GM_LUT_BYTES + 256;
    return need > GM_MIN_SMEM ? need : GM_MIN_SMEM;
}

constexpr int64_t GM_COUNTER_BYTES = 4096;   // head of the split-K workspace: arrival counters

// Tile height and K split for a shape.  Few weight tiles (decode shapes, narrow layers) leave SMs idle, so K
// is cut into ranges until about two small CTAs (or one large) per SM exist; each range keeps >= 4 K blocks.
static void gemm_plan(int64_t M, int64_t N, int64_t K, int* TM_out, int* splits_out) {
    int TM = 256;
    while (TM > 32 && TM / 2 >= M) TM /= 2;         // 32, 64, 128 or 256 activation rows per CTA
    const int64_t ctas = ((N + GM_BM - 1) / GM_BM) * ((M + TM - 1) / TM);
    const int64_t target = TM <= 64 ? GM_MAX_CTAS_SPLIT : GM_MAX_CTAS_SPLIT / 2;
    int64_t splits = target / ctas;
    if (splits > K / 64 / 4) splits = K / 64 / 4;
    if (splits < 1) splits = 1;
    const char* e = getenv("NF4_GEMM_SPLITS");
    const int forced = e ? atoi(e) : -1;
    if (forced >= 1) splits = forced < K / 64 ? forced : K / 64;
    *TM_out = TM;
    *splits_out = (int)splits;
}

static int64_t gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M < 1 || N < 1 || K < 64) return 0;
    int TM, splits;
    gemm_plan(M, N, K, &TM, &splits);
    if (splits == 1) return 0;
    const int64_t groups = ((N + GM_BM - 1) / GM_BM) * ((M + TM - 1) / TM);
    return GM_COUNTER_BYTES + groups * splits * TM * 128 * 4;
}

// smallest M the dispatcher sends to this kernel instead of the GEMV (NF4_GEMM_MIN_M overrides)
int gemm_min_m() {
    const char* e = getenv("NF4_GEMM_MIN_M");
    const int v = e ? atoi(e) : 9;
    return v < 1 ? 1 : v;
}

bool gemm_supported(int64_t M, int64_t K, int64_t N, int blocksize, int dtype, const void* x, const void* packed,
                    const void* absmax, const void* y) {
    (void)y;
    return M >= gemm_min_m() && dtype == NF4_BF16 && blocksize == 64 && K >= 64 && K % 64 == 0 && N >= 1 && M < (1ll << 30) &&
           N < (1ll << 30) && K < (1ll << 24) && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
           reinterpret_cast<uintptr_t>(packed) % 16 == 0 && reinterpret_cast<uintptr_t>(absmax) % 4 == 0;
}

struct GemmExtras {
    const void* residual = nullptr;
    int epilogue = 0;
    int pdl = 0;
    void* workspace = nullptr;
    int64_t workspace_bytes = 0;
};

static int gemm_tcgen05(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax, const float* code16,
                        int64_t N, const void* bias, void* y, const GemmExtras& ex, cudaStream_t stream) {
    GmEncodeFn enc = gm_encode_fn();
    NF4_REQUIRE(enc, NF4_ERR_CUDA, "gemm: cuTensorMapEncodeTiled is not available from this driver");
    GemmParams p;
    int TM, splits;
    gemm_plan(M, N, K, &TM, &splits);
    const int64_t ntiles = (N + GM_BM - 1) / GM_BM, mtiles = (M + TM - 1) / TM;
    // without (enough) workspace the K split is dropped: same sums, fewer CTAs
    if (splits > 1 && (!ex.workspace || ex.workspace_bytes < GM_COUNTER_BYTES + ntiles * mtiles * splits * TM * 128 * 4 ||
                       ntiles * mtiles * 4 > GM_COUNTER_BYTES || reinterpret_cast<uintptr_t>(ex.workspace) % 16 != 0))
        splits = 1;
    p.TM = TM;
    p.splits = splits;
    p.tmem_cols = 32;                               // a power of two >= 32
    while (p.tmem_cols < TM + GM_STAGES * GM_A_COLS) p.tmem_cols *= 2;
    p.absmax = absmax; p.code16 = code16; p.bias = bias; p.y = y;
    p.residual = ex.residual; p.epilogue = ex.epilogue; p.pdl = ex.pdl;
    p.counters = static_cast<unsigned*>(ex.workspace);
    p.partials = ex.workspace ? reinterpret_cast<float*>(static_cast<uint8_t*>(ex.workspace) + GM_COUNTER_BYTES) : nullptr;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.KB = (int)(K / 64);
    const cuuint32_t estr[2] = {1, 1};
    {
        const cuuint64_t dim[2] = {(cuuint64_t)(K / 2), (cuuint64_t)N};
        const cuuint64_t str[1] = {(cuuint64_t)(K / 2)};
        const cuuint32_t box[2] = {128, (cuuint32_t)GM_BM};
        CUresult r = enc(&p.wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(packed), dim, str, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        NF4_REQUIRE(r == CUDA_SUCCESS, NF4_ERR_CUDA, "gemm: cuTensorMapEncodeTiled(weights) failed with %d", (int)r);
    }
    {
        const cuuint64_t dim[2] = {(cuuint64_t)K, (cuuint64_t)M};
        const cuuint64_t str[1] = {(cuuint64_t)K * 2};
        const cuuint32_t box[2] = {64, (cuuint32_t)TM};
        CUresult r = enc(&p.xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dim, str, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        NF4_REQUIRE(r == CUDA_SUCCESS, NF4_ERR_CUDA, "gemm: cuTensorMapEncodeTiled(activations) failed with %d", (int)r);
    }
    static bool configured[64] = {false};
    int dev = 0;
    NF4_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        NF4_CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm_smem_bytes(256)));
        configured[dev] = true;
    }
    dim3 grid((unsigned)ntiles, (unsigned)(mtiles * splits));
    NF4_REQUIRE(grid.y <= 65535, NF4_ERR_LIMIT, "gemm: M=%lld too large", (long long)M);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(GM_THREADS);
    cfg.dynamicSmemBytes = (size_t)gemm_smem_bytes(TM);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ex.pdl ? 1 : 0;
    NF4_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel, p));
    return NF4_OK;
}

}  // namespace nf4

using namespace nf4;

extern "C" int64_t nf4_b200_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) { return gemm_workspace_bytes(M, N, K); }

extern "C" int nf4_b200_gemm(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                             const float* code16, int64_t N, const void* bias, void* y, int dtype, void* workspace,
                             int64_t workspace_bytes, void* stream) {
    NF4_REQUIRE(x && packed && absmax && code16 && y, NF4_ERR_ARG, "gemm: null pointer");
    NF4_REQUIRE(M >= 1 && N >= 1, NF4_ERR_ARG, "gemm: M=%lld N=%lld", (long long)M, (long long)N);
    NF4_REQUIRE(K >= 64 && K % 64 == 0, NF4_ERR_ARG, "gemm: K=%lld must be a positive multiple of 64", (long long)K);
    NF4_REQUIRE(dtype == NF4_BF16 || dtype == NF4_F16, NF4_ERR_ARG, "gemm: dtype code %d is not fp16/bf16", dtype);
    if (int rc = check_device()) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (gemm_supported(M >= gemm_min_m() ? M : gemm_min_m(), K, N, 64, dtype, x, packed, absmax, y)) {
        GemmExtras ex;
        ex.workspace = workspace;
        ex.workspace_bytes = workspace_bytes;
        return gemm_tcgen05(x, M, K, packed, absmax, code16, N, bias, y, ex, s);
    }
    // fp16, or pointers the TMA path cannot take: the GEMV kernel, 16 activation rows at a time
    NF4_REQUIRE(gemv_supported(M < 16 ? M : 16, K, N, 64, dtype, x, packed, absmax), NF4_ERR_ALIGN,
                "gemm: x must be 16-byte aligned, packed 8-byte aligned");
    for (int64_t m0 = 0; m0 < M; m0 += 16) {
        const int64_t mc = (M - m0) < 16 ? (M - m0) : 16;
        int rc = nf4_b200_gemv(static_cast<const uint8_t*>(x) + m0 * K * 2, mc, K, packed, absmax, code16, N, bias,
                               static_cast<uint8_t*>(y) + m0 * N * 2, dtype, stream);
        if (rc) return rc;
    }
    return NF4_OK;
}

extern "C" int nf4_b200_gemm_decode(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                                    const float* code16, int64_t N, const void* residual, void* y, int epilogue,
                                    void* workspace, int64_t workspace_bytes, int flags, void* stream) {
    NF4_REQUIRE(x && packed && absmax && code16 && y, NF4_ERR_ARG, "gemm_decode: null pointer");
    NF4_REQUIRE(M >= 1 && N >= 1, NF4_ERR_ARG, "gemm_decode: M=%lld N=%lld", (long long)M, (long long)N);
    NF4_REQUIRE(K >= 64 && K % 64 == 0, NF4_ERR_ARG, "gemm_decode: K=%lld must be a positive multiple of 64", (long long)K);
    NF4_REQUIRE(epilogue == 0 || (epilogue == 1 && N % 2 == 0 && !residual), NF4_ERR_ARG,
                "gemm_decode: epilogue %d (1 needs an even N and no residual)", epilogue);
    NF4_REQUIRE(reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(packed) % 16 == 0, NF4_ERR_ALIGN,
                "gemm_decode: x and packed must be 16-byte aligned");
    NF4_REQUIRE(M < (1ll << 30) && N < (1ll << 30) && K < (1ll << 24), NF4_ERR_LIMIT, "gemm_decode: extent too large");
    if (int rc = check_device()) return rc;
    GemmExtras ex;
    ex.residual = residual;
    ex.epilogue = epilogue;
    ex.pdl = flags & 1;
    ex.workspace = workspace;
    ex.workspace_bytes = workspace_bytes;
    return gemm_tcgen05(x, M, K, packed, absmax, code16, N, nullptr, y, ex, static_cast<cudaStream_t>(stream));
}
