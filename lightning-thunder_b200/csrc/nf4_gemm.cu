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
// PAIR (template flag; 256-row tiles, no K split, an even number of weight tiles): two CTAs of a cluster -- two
// adjacent weight tiles, the same 256 activation rows -- run as one `cta_group::2` MMA of 256 weight rows.  Each
// CTA dequantises its own 128 rows into its own tensor memory and loads only HALF of the activation tile (128 rows,
// 16 KB per K block instead of 32 KB) into its shared memory; the leader (cluster rank 0) issues every MMA, which
// reads the activation halves from both CTAs.  Per CTA that halves the L2 -> shared-memory traffic (16 instead of
// 32 KB per K block) and doubles the ring to six stages.  MEASURED 3-10 % SLOWER than one CTA per tile (the period
// of a K-block group is set by dequantise -> hand-off -> multiply -> hand-off, and every hand-off now crosses the
// pair), so it is off unless NF4_GEMM_PAIR=1.  Hand-offs across the pair: the peer's activation loads
// complete on the LEADER's `full` barrier (cp.async.bulk.tensor with .cta_group::2, no multicast), the peer's
// dequant warps arrive on the leader's `a_ready`, and the leader's tcgen05.commit arrives on `done` / `acc_done`
// of both CTAs (.multicast::cluster).
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
int gemm_clear_error() {
    const unsigned int zero[4] = {0u, 0u, 0u, 0u};
    NF4_CUDA_TRY(cudaMemcpyToSymbol(g_gemm_error, zero, sizeof(zero)));
    return NF4_OK;
}

constexpr int GM_DQ_WARPS = 16;          // dequant warps: four threads per weight row (a quarter block each)
constexpr int GM_THREADS = (3 + GM_DQ_WARPS) * 32;   // activation producer, MMA, dequant (the first 4 also run the epilogue), weight producer
constexpr int GM_WPRODUCER = 2 + GM_DQ_WARPS;        // warp index of the weight producer
constexpr int GM_BM = 128;               // weight rows per CTA (UMMA M)
constexpr int GM_MAX_STAGES = 8;         // activation stages: 8 (tiles up to 64 rows), 4 (128 rows) or 3 (256 rows)
constexpr int GM_DONE = 8;               // ring of "MMAs up to here have completed" barriers, one per release unit
constexpr int GM_A_COLS = 32;            // TMEM columns of one K block of weights: 64 bf16 per row, two per column
constexpr int GM_GKB = 4;                // K blocks per weight group in TMEM (a whole packed stage)
constexpr int GM_GROUPS = 2;             // weight groups in TMEM: one converts while one multiplies.  Four groups of 2 blocks (a hand-off
                                         // after every 2 blocks, more slack between the two sides) measured 7 % SLOWER: the extra
                                         // tcgen05.wait::st + arrival per packed stage costs the dequant warps more than the slack gives
constexpr int GM_A_COL0 = 256;           // accumulator in TMEM columns [0, 256), weight groups in [256, 512)
constexpr int GM_TMEM_COLS = 512;
constexpr int GM_MAX_WSTAGES = 4;        // packed-weight stages, each GM_WKB K blocks deep: 4, or 3 for 256-row tiles
constexpr int GM_WKB = 4;                // K blocks per packed-weight stage: 4 x 32 B = one 128-byte swizzle row
constexpr int GM_PK_BYTES = GM_BM * 128; // one packed-weight stage
constexpr int GM_AM_BYTES = GM_BM * 16;  // its absmax: 4 floats per row
constexpr uint32_t GM_LUT_WINDOW = 65536;  // byte -> (fp32, fp32): 256 entries x 32 lanes x 8 B, 64 KB aligned in the shared window
constexpr uint32_t GM_LOW_BASE = 2048;     // buffers below the window start here (the dynamic region starts at or below it)
constexpr int GM_SM_TARGET = 148;        // split K until about one CTA per SM exists
constexpr unsigned long long GM_WAIT_LIMIT_NS = 200ull * 1000 * 1000;

struct alignas(64) GemmParams {
    CUtensorMap wmap;     // packed codes uint8 [N][K/2], box 128 B x 128 rows, SWIZZLE_128B
    CUtensorMap xmap;     // activations bf16 [M][K], box 64 x TM, SWIZZLE_128B
    CUtensorMap amap;     // absmax fp32 [N][K/64], box 4 x 128 (used when K/64 is a multiple of 4)
    const float* absmax;
    const float* code16;
    const void* bias;
    const void* residual; // bf16 [M][N] added in the epilogue, or null
    void* y;
    float* partials;      // split K: fp32 [group][split][TM][128]
    unsigned* counters;   // split K: one arrival counter per (weight tile, activation tile); zero between launches
    int M, N, K, KB;
    int TM;               // activation rows per CTA: multiple of 16, 32..256
    int splits;           // K is cut into this many ranges, one CTA each
    int epilogue;         // 0: y[m][n];  1: rows are (gate, up) pairs, y[m][n/2] = silu(gate) * up
    int pdl;              // programmatic dependent launch: weights may be fetched before the upstream grid ends
    int stages, wstages;  // ring depths
    int ru_shift;         // log2 of the K blocks per release unit: the MMA thread commits once per unit (a commit stalls it
                          // for about as long as two MMAs), which frees the unit's activation stages and tells
                          // the dequant warps how far the tensor core has got
    // shared-window addresses (the table takes [64K, 128K); the host lays the rest out around it)
    uint32_t b_addr[GM_MAX_STAGES];    // activation stages, 1024-byte aligned
    uint32_t w_addr[GM_MAX_WSTAGES];   // packed-weight stages, 1024-byte aligned
    uint32_t am_addr[GM_MAX_WSTAGES];  // absmax of a packed stage: 128 rows x 4 floats
    int am_tma;                        // absmax travels with the packed weights (else it is loaded from global)
    uint32_t bar_addr;                 // mbarriers + 16 bytes of flags
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
// Bounded wait.  The hot path is a plain poll of the barrier; only a wait that has already lasted thousands
// of polls starts reading the timer and the CTA's abort flag (both are slow enough to show in a hand-off).
__device__ __noinline__ void gm_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, int iter) {
    if (*abort_flag) return;
    const unsigned long long t0 = gm_global_ns();
    while (true) {
        for (int spin = 0; spin < 256; ++spin)
            if (gm_mbar_try_wait(bar, parity)) return;
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
__device__ __forceinline__ void gm_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, int iter) {
#pragma unroll 1
    for (int spin = 0; spin < 4096; ++spin)
        if (gm_mbar_try_wait(bar, parity)) return;
    gm_wait_slow(bar, parity, abort_flag, code, iter);
}
__device__ __forceinline__ void gm_tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}

// table lookup: the packed byte `sel` of `word` becomes bits 8..15 of the 64 KB aligned window address
template <int SEL>
__device__ __forceinline__ void gm_lookup(uint32_t word, uint32_t window_lane, float& first, float& second) {
    const uint32_t addr = __byte_perm(word, window_lane, 0x7604 | (SEL << 4));
    asm("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(first), "=f"(second) : "r"(addr));
}
__device__ __forceinline__ uint32_t gm_scale_pack(float first, float second, float am) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(first * am, second * am);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// D[tmem] (+)= A[tmem] . B[smem]^T, 128 x N x 16, bf16 operands, fp32 accumulator
__device__ __forceinline__ void gm_mma(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.u32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// the mbarrier gets one arrival once every MMA issued so far by this thread has completed
__device__ __forceinline__ void gm_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- two-CTA (cta_group::2) forms -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t gm_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t gm_mapa(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void gm_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void gm_mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// TMA load into this CTA's shared memory whose bytes complete on a barrier that may live in the pair's other CTA
__device__ __forceinline__ void gm_tma_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(cluster_bar) : "memory");
}
// D[tmem of both CTAs] (+)= A[tmem of both CTAs] . B[smem halves of both CTAs]^T, 256 x N x 16
__device__ __forceinline__ void gm_mma_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    const uint32_t z = 0u;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.u32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(z) : "memory");
}
// the barrier at this shared-memory offset in BOTH CTAs gets one arrival once every MMA issued so far has completed
__device__ __forceinline__ void gm_commit_pair(uint32_t bar) {
    const unsigned short mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
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
__device__ __forceinline__ uint32_t gm_instr_desc(int n, int m = GM_BM) {
    uint32_t d = 0;
    d |= 1u << 4;                      // D format f32
    d |= 1u << 7;                      // A format bf16
    d |= 1u << 10;                     // B format bf16
    d |= (uint32_t)(n >> 3) << 17;     // N >> 3
    d |= (uint32_t)(m >> 4) << 24;     // M >> 4 (256 for a CTA pair: 128 rows in each CTA)
    return d;
}

template <bool PAIR>
__global__ void __launch_bounds__(GM_THREADS, 1) gemm_tcgen05_kernel(const __grid_constant__ GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int TM = p.TM;
    const uint32_t cta_rank = PAIR ? gm_cluster_rank() : 0u;     // 0: the CTA that issues the pair's MMAs
    const int TML = PAIR ? TM >> 1 : TM;                          // activation rows this CTA loads per K block
    const int b_bytes = TML * 128;
    const int NS = p.stages, NW = p.wstages;

    // The host laid the buffers out in shared-window addresses around the table's window [64K, 128K),
    // assuming the dynamic region starts at or below GM_LOW_BASE.
    // Shared-memory addresses.  The host laid the buffers out as offsets into the CTA's shared window.  Outside a
    // cluster (and in rank 0 of one) the window starts at address 0 and an offset IS the address.  In rank 1 of a
    // cluster the window starts higher (the address of a shared variable carries the CTA's rank above the offset
    // bits; a window is smaller than 2^18 bytes) and a bare offset is not an address of this CTA at all -- a plain
    // ld.shared with it traps.  So every address below is rebased by W, this CTA's window base; `to_leader`
    // turns an address of this CTA into the leader's (for barriers the pair shares).
    const uint32_t base_full = gm_smem_u32(smem);
    const uint32_t s0 = base_full & 0x3ffffu;          // offset of the dynamic region inside the window
    const uint32_t W = PAIR ? base_full - s0 : 0u;
    const uint32_t to_leader = PAIR ? gm_mapa(base_full, 0u) - base_full : 0u;
    if (s0 > GM_LOW_BASE) {
        if (tid == 0 && atomicCAS(&g_gemm_error[0], 0u, 10u) == 0u) g_gemm_error[1] = s0;
        return;
    }
    const uint32_t full0 = p.bar_addr + W, done0 = full0 + 8 * GM_MAX_STAGES, aready0 = done0 + 8 * GM_DONE,
                   accdone = aready0 + 8 * GM_GROUPS, wfull0 = accdone + 8,
                   wempty0 = wfull0 + 8 * GM_MAX_WSTAGES, flags0 = wempty0 + 8 * GM_MAX_WSTAGES;
    const uint32_t desc0 = flags0 + 16;              // activation descriptors per stage (8 x 8 bytes)
    const int ru_shift = p.ru_shift, ru_mask = (1 << ru_shift) - 1;
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(smem + (flags0 - W - s0));
    volatile int* const abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* const last_flag = abort_flag + 1;

    const int n0 = blockIdx.x * GM_BM;
    const int mtile = blockIdx.y / p.splits;
    const int split = blockIdx.y - mtile * p.splits;
    const int m0 = mtile * TM;
    // this CTA's range of 64-element K blocks (never empty: splits <= KB)
    // (whole groups of GM_WKB blocks when absmax comes by TMA: its box must start 16-byte aligned)
    const int units = p.am_tma ? p.KB / GM_WKB : p.KB, unit = p.am_tma ? GM_WKB : 1;
    const int kb_begin = (int)((int64_t)units * split / p.splits) * unit;
    const int kb_end = (int)((int64_t)units * (split + 1) / p.splits) * unit;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) gm_mbar_init(full0 + 8 * s, 1);
        for (int s = 0; s < GM_DONE; ++s) gm_mbar_init(done0 + 8 * s, 1);   // tcgen05.commit after a unit's MMAs
        for (int g = 0; g < GM_GROUPS; ++g) gm_mbar_init(aready0 + 8 * g, (PAIR ? 2 : 1) * GM_DQ_WARPS);   // one arrival per dequant warp (of both CTAs)
        for (int s = 0; s < NW; ++s) {
            gm_mbar_init(wfull0 + 8 * s, 1);
            gm_mbar_init(wempty0 + 8 * s, GM_DQ_WARPS);   // every dequant warp has read its rows
        }
        gm_mbar_init(accdone, 1);
        *abort_flag = 0;
        for (int s = 0; s < NS; ++s) {
            const uint64_t d = gm_smem_desc(p.b_addr[s]);
            asm volatile("st.shared.b64 [%0], %1;" ::"r"(desc0 + 8 * s), "l"(d) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // TMEM allocation by one full warp; the base address lands in shared memory.  In a pair each CTA
        // allocates its own tensor memory (all 512 columns of an empty TMEM: the same base in both CTAs)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(flags0), "r"(GM_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp >= 2 && warp < GM_WPRODUCER) {
        // byte -> (float(bf16(code[hi])), float(bf16(code[lo]))), one copy per lane (conflict-free lookups):
        // entry e of lane l at window + e * 256 + l * 8
        const float mine = __bfloat162float(__float2bfloat16_rn(__ldg(p.code16 + (lane & 15))));
        for (int e = warp - 2; e < 256; e += GM_DQ_WARPS) {
            const float first = __shfl_sync(0xffffffffu, mine, e >> 4), second = __shfl_sync(0xffffffffu, mine, e & 15);
            asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(W + GM_LUT_WINDOW + (uint32_t)(e * 256 + lane * 8)), "f"(first), "f"(second) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (PAIR) gm_cluster_sync();      // the other CTA's barriers exist before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;
    if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ------------------------------ activation producer -----------------------------------
        int slot = 0;
        if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");   // x comes from the upstream grid
        for (int kb = kb_begin; kb < kb_end; ++kb) {
            const int i = kb - kb_begin;
            if (i >= NS) {      // the stage's previous K block belongs to unit u: wait until that unit's MMAs are done
                const int u = (i - NS) >> ru_shift;
                gm_wait(done0 + 8 * (u % GM_DONE), (uint32_t)((u / GM_DONE) & 1), abort_flag, 6, kb);
            }
            if (lane == 0) {
                const uint32_t fb = full0 + 8 * slot;
                if (PAIR) {
                    // both halves of the stage complete on the leader's barrier, which the leader arms for both
                    if (cta_rank == 0) gm_mbar_expect_tx(fb, 2u * (uint32_t)b_bytes);
                    gm_tma_2d_pair(W + p.b_addr[slot], &p.xmap, kb * 64, m0 + (int)cta_rank * TML, fb + to_leader);
                } else {
                    gm_mbar_expect_tx(fb, (uint32_t)b_bytes);
                    gm_tma_2d(W + p.b_addr[slot], &p.xmap, kb * 64, m0, fb);
                }
            }
            __syncwarp();
            if (++slot == NS) slot = 0;
        }
    } else if (warp == GM_WPRODUCER) {
        // -------------------------------- weight producer --------------------------------------
        // packed weights: one box of 128 rows x 128 bytes (a group of GM_WKB K blocks) per weight stage, running
        // up to `wstages` groups ahead of the dequant warps whatever the activation ring does; the weights do
        // not depend on the upstream grid, so nothing here waits for it
        int wslot = 0;
        uint32_t wparity = 0;
        for (int kb = kb_begin; kb < kb_end; kb += GM_WKB) {
            gm_wait(wempty0 + 8 * wslot, wparity ^ 1u, abort_flag, 9, kb);
            if (lane == 0) {
                gm_mbar_expect_tx(wfull0 + 8 * wslot, (uint32_t)(GM_PK_BYTES + (p.am_tma ? GM_AM_BYTES : 0)));
                gm_tma_2d(W + p.w_addr[wslot], &p.wmap, kb * 32, n0, wfull0 + 8 * wslot);
                if (p.am_tma) gm_tma_2d(W + p.am_addr[wslot], &p.amap, kb, n0, wfull0 + 8 * wslot);
            }
            __syncwarp();
            if (++wslot == NW) { wslot = 0; wparity ^= 1u; }
        }
    } else if (warp == 1 && cta_rank == 0) {
        // ------------------------------------ MMA issuer ---------------------------------------
        // (PAIR: only the leader's; its MMAs run on both CTAs' tensor cores)
        // per group of GM_GKB K blocks: one wait for the dequantised weights, 4 MMAs per K block as its
        // activations land, one commit per K block (frees the activation stage) and one per group.
        // This warp's instruction stream is serial and sits on the critical path of small tiles, so the
        // descriptors are built once and the loop body is kept short.
        const uint32_t idesc = PAIR ? gm_instr_desc(TM, 2 * GM_BM) : gm_instr_desc(TM);
        int slot = 0, g = 0, i = 0;              // i: K block index inside this CTA's range
        uint32_t parity = 0, gparity = 0;
        uint32_t accumulate = 0u;
        const int nkb = kb_end - kb_begin;
        for (int kb0 = kb_begin; kb0 < kb_end; kb0 += GM_GKB) {
            gm_wait(aready0 + 8 * g, gparity, abort_flag, 7, kb0);     // the group's weights are in TMEM
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int nblk = min(GM_GKB, kb_end - kb0);
            uint32_t a_tmem = tmem_d + (uint32_t)(GM_A_COL0 + g * GM_GKB * GM_A_COLS);
            for (int j = 0; j < nblk; ++j, a_tmem += GM_A_COLS, ++i) {
                gm_wait(full0 + 8 * slot, parity, abort_flag, 5, kb0 + j);  // activations landed
                if (lane == 0) {
                    uint64_t bdesc;
                    asm volatile("ld.shared.b64 %0, [%1];" : "=l"(bdesc) : "r"(desc0 + 8 * slot));
                    // 16 K elements per instruction: 8 TMEM columns of the weights, 32 bytes (+2 in the
                    // descriptor's address field) inside the activations' swizzle atom
                    if (PAIR) {
                        gm_mma_pair(tmem_d, a_tmem, bdesc, idesc, accumulate);
                        gm_mma_pair(tmem_d, a_tmem + 8u, bdesc + 2u, idesc, 1u);
                        gm_mma_pair(tmem_d, a_tmem + 16u, bdesc + 4u, idesc, 1u);
                        gm_mma_pair(tmem_d, a_tmem + 24u, bdesc + 6u, idesc, 1u);
                    } else {
                        gm_mma(tmem_d, a_tmem, bdesc, idesc, accumulate);
                        gm_mma(tmem_d, a_tmem + 8u, bdesc + 2u, idesc, 1u);
                        gm_mma(tmem_d, a_tmem + 16u, bdesc + 4u, idesc, 1u);
                        gm_mma(tmem_d, a_tmem + 24u, bdesc + 6u, idesc, 1u);
                    }
                    // one commit per release unit (and at the end of the range)
                    if (((i + 1) & ru_mask) == 0 || i == nkb - 1) {
                        const uint32_t db = done0 + 8 * ((i >> ru_shift) & (GM_DONE - 1));
                        if (PAIR) gm_commit_pair(db); else gm_commit(db);
                    }
                }
                accumulate = 1u;
                if (++slot == NS) { slot = 0; parity ^= 1u; }
            }
            if (++g == GM_GROUPS) { g = 0; gparity ^= 1u; }
        }
        if (lane == 0) { if (PAIR) gm_commit_pair(accdone); else gm_commit(accdone); }
        __syncwarp();
    } else if (warp == 1) {
        // the other CTA's MMA warp has nothing to issue; it releases tensor memory at the end
    } else {
        // ------------------------------------ dequant warps -------------------------------------
        // a warp may touch only the TMEM lane quarter warp % 4, so rows follow that numbering
        const int q = warp & 3;
        const int r = q * 32 + lane;            // weight row inside the tile = TMEM lane
        const int part = (warp - 2) >> 2;       // which quarter of the row's 64-block: packed bytes [8*part, 8*part+8)
        const int grow = n0 + r;
        const uint32_t window_lane = (W + GM_LUT_WINDOW) | (uint32_t)(lane << 3);
        const float* const am_row = p.absmax + (int64_t)(grow < p.N ? grow : 0) * p.KB;
        const bool row_ok = grow < p.N;
        // this thread's 8 bytes of K block j of a packed stage: 16-byte chunk 2j + part/2 at its swizzled place
        const uint32_t pk_off = (uint32_t)(r * 128 + (part & 1) * 8);
        const int rsw = r & 7, chunk0 = part >> 1;
        const uint32_t tcol = tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)(GM_A_COL0 + part * 8);
        int g = 0, wslot = 0;
        uint32_t gparity = 0, wparity = 0;
        // absmax of a group's K blocks is fetched one group ahead
        float am_nxt[GM_WKB];
#pragma unroll
        for (int j = 0; j < GM_WKB; ++j) am_nxt[j] = (!p.am_tma && row_ok && kb_begin + j < kb_end) ? __ldg(am_row + kb_begin + j) : 0.0f;
        for (int kb0 = kb_begin; kb0 < kb_end; kb0 += GM_WKB) {
            float am[GM_WKB];
            if (!p.am_tma) {
#pragma unroll
                for (int j = 0; j < GM_WKB; ++j) {
                    am[j] = am_nxt[j];
                    am_nxt[j] = (row_ok && kb0 + GM_WKB + j < kb_end) ? __ldg(am_row + kb0 + GM_WKB + j) : 0.0f;
                }
            }
            gm_wait(wfull0 + 8 * wslot, wparity, abort_flag, 5, kb0);   // packed bytes (and absmax) landed
            if (p.am_tma)
                asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(am[0]), "=f"(am[1]), "=f"(am[2]), "=f"(am[3])
                             : "r"(W + p.am_addr[wslot] + (uint32_t)(r * 16)));
            uint2 w[GM_WKB];
#pragma unroll
            for (int j = 0; j < GM_WKB; ++j)
                asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(w[j].x), "=r"(w[j].y)
                             : "r"(W + p.w_addr[wslot] + pk_off + (uint32_t)(((2 * j + chunk0) ^ rsw) << 4)));
            // the packed stage feeds GM_WKB / GM_GKB groups; each is handed to the tensor core as soon as it is in TMEM
#pragma unroll
            for (int h = 0; h < GM_WKB / GM_GKB; ++h) {
                if (kb0 + h * GM_GKB >= kb_end) break;          // the range ends inside this packed stage
                const int gi = (kb0 - kb_begin) / GM_GKB + h;
                if (gi >= GM_GROUPS) {   // these TMEM columns held group gi - GM_GROUPS: its last K block's unit must be done
                    const int u = ((gi - GM_GROUPS) * GM_GKB + GM_GKB - 1) >> ru_shift;
                    gm_wait(done0 + 8 * (u % GM_DONE), (uint32_t)((u / GM_DONE) & 1), abort_flag, 6, kb0);
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int jj = 0; jj < GM_GKB; ++jj) {
                    const int j = h * GM_GKB + jj;
                    // 8 packed bytes -> 16 weights: all 8 lookups in flight, then scale and round.  Blocks past the
                    // end of the range convert whatever the box brought; no MMA reads them.
                    float f[16];
                    gm_lookup<0>(w[j].x, window_lane, f[0], f[1]);
                    gm_lookup<1>(w[j].x, window_lane, f[2], f[3]);
                    gm_lookup<2>(w[j].x, window_lane, f[4], f[5]);
                    gm_lookup<3>(w[j].x, window_lane, f[6], f[7]);
                    gm_lookup<0>(w[j].y, window_lane, f[8], f[9]);
                    gm_lookup<1>(w[j].y, window_lane, f[10], f[11]);
                    gm_lookup<2>(w[j].y, window_lane, f[12], f[13]);
                    gm_lookup<3>(w[j].y, window_lane, f[14], f[15]);
                    uint32_t out[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) out[i] = gm_scale_pack(f[2 * i], f[2 * i + 1], am[j]);
                    // 8 columns (16 consecutive K elements) of this thread's lane
                    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                                     ::"r"(tcol + (uint32_t)((g * GM_GKB + jj) * GM_A_COLS)), "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3]),
                                       "r"(out[4]), "r"(out[5]), "r"(out[6]), "r"(out[7]) : "memory");
                }
                // the group is in TMEM: hand it over
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) gm_mbar_arrive_cluster(aready0 + 8 * g + to_leader);    // the leader waits for both CTAs' weights
                    else gm_mbar_arrive(aready0 + 8 * g);
                }
                if (++g == GM_GROUPS) { g = 0; gparity ^= 1u; }
            }
            // the packed stage has been consumed
            __syncwarp();
            if (lane == 0) gm_mbar_arrive(wempty0 + 8 * wslot);
            if (++wslot == NW) { wslot = 0; wparity ^= 1u; }
        }
        if (warp >= 6) goto done;               // the epilogue needs one warp per TMEM lane quarter
        // ------------------------------------ epilogue ------------------------------------------
        gm_wait(accdone, 0u, abort_flag, 8, kb_end);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int gn = grow;                    // accumulator lane = weight row
        const int mlim = min(TM, p.M - m0);     // activation rows of this tile that exist
        const int group = mtile * gridDim.x + blockIdx.x;
        const uint32_t tacc = tmem_d + ((uint32_t)(q * 32) << 16);
        __nv_bfloat16* const y = static_cast<__nv_bfloat16*>(p.y);
        if (p.splits == 1 && p.epilogue == 0 && !p.residual && mlim > 16 && (p.N & 7) == 0 &&
            (reinterpret_cast<uintptr_t>(p.y) & 15) == 0) {
            // Tall tiles: round to bf16, transpose through shared memory (the activation stages are idle now:
            // every MMA has completed), then store rows of y 16 bytes per lane.  Stage s holds rows
            // [s * TM/2, (s+1) * TM/2) of the tile, 256 bytes (128 columns of y) each.
            const float bias = (p.bias && gn < p.N) ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[gn]) : 0.0f;
            const int rps_shift = PAIR ? 6 : (TM == 256 ? 7 : TM == 128 ? 6 : TM == 64 ? 5 : 4);   // rows of y per stage buffer: stage bytes / 256
            const int rps_mask = (1 << rps_shift) - 1;
            for (int c0 = 0; c0 < mlim; c0 += 16) {
                uint32_t v[16];
                gm_tmem_ld16(tacc + (uint32_t)c0, v);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int m = c0 + j;
                    const uint32_t dst = W + p.b_addr[m >> rps_shift] + (uint32_t)((m & rps_mask) * 256 + r * 2);
                    const __nv_bfloat16 h = __float2bfloat16_rn(__uint_as_float(v[j]) + bias);
                    asm volatile("st.shared.b16 [%0], %1;" ::"r"(dst), "h"(*reinterpret_cast<const unsigned short*>(&h)) : "memory");
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int et = tid - 64;                      // 0..127 over the four epilogue warps
            const int chunk = et & 15;                    // 16-byte chunk of a 256-byte row
            const bool col_ok = n0 + chunk * 8 < p.N;
            for (int m = et >> 4; m < mlim; m += 8) {
                const uint32_t src = W + p.b_addr[m >> rps_shift] + (uint32_t)((m & rps_mask) * 256 + chunk * 16);
                uint4 d;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(d.x), "=r"(d.y), "=r"(d.z), "=r"(d.w) : "r"(src));
                if (col_ok) *reinterpret_cast<uint4*>(y + (int64_t)(m0 + m) * p.N + n0 + chunk * 8) = d;
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            goto done;
        }
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
    if (PAIR) gm_cluster_sync();      // neither CTA leaves (or frees tensor memory) while the other may still touch it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(GM_TMEM_COLS) : "memory");
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

// Shared-memory map in shared-window addresses: the lookup table owns [64K, 128K); activation stages, packed
// stages and the barriers are dealt, 1024-byte aligned, first into [GM_LOW_BASE, 64K), then from 128K up.
// Returns the dynamic shared memory to request (the region starts at or below GM_LOW_BASE).
static int gemm_layout(int TM, bool pair, GemmParams* p) {
    uint32_t low = GM_LOW_BASE, high = 2 * GM_LUT_WINDOW;
    auto place = [&](uint32_t bytes) {
        const uint32_t size = (bytes + 1023u) & ~1023u;
        uint32_t addr;
        if (low + size <= GM_LUT_WINDOW) { addr = low; low += size; }
        else { addr = high; high += size; }
        return addr;
    };
    // activation ring and release unit: 8 stages freed 4 at a time for small tiles, 4 freed in pairs for
    // 128-row tiles, 3 freed one by one for 256-row tiles (all that fits beside the table)
    // (a CTA of a pair holds half of the activation tile per stage: six stages of 16 KB in the same space)
    int stages = TM > 128 ? 3 : TM > 64 ? 4 : 8, ru = TM > 128 ? 1 : TM > 64 ? 2 : 4;
    if (pair) { stages = 6; ru = 1; }
    const int wstages = TM > 128 ? 3 : GM_MAX_WSTAGES;
    if (p) { p->stages = stages; p->wstages = wstages; p->ru_shift = ru == 4 ? 2 : ru == 2 ? 1 : 0; }
    for (int s = 0; s < stages; ++s) {
        const uint32_t a = place((uint32_t)(pair ? TM / 2 : TM) * 128u);
        if (p) p->b_addr[s] = a;
    }
    for (int s = 0; s < wstages; ++s) {
        const uint32_t a = place((uint32_t)GM_PK_BYTES);
        if (p) p->w_addr[s] = a;
    }
    for (int s = 0; s < wstages; ++s) {
        const uint32_t a = place((uint32_t)GM_AM_BYTES);
        if (p) p->am_addr[s] = a;
    }
    const uint32_t bars = place(512);
    if (p) p->bar_addr = bars;
    return (int)high;
}

constexpr int64_t GM_COUNTER_BYTES = 4096;   // head of the split-K workspace: arrival counters

// Tile height and K split for a shape.  Few weight tiles (decode shapes, narrow layers) leave SMs idle, so K
// is cut into ranges until about one CTA per SM exists.
static void gemm_plan(int64_t M, int64_t N, int64_t K, int* TM_out, int* splits_out) {
    int TM = 256;
    while (TM > 32 && TM / 2 >= M) TM /= 2;         // 32, 64, 128 or 256 activation rows per CTA
    if (const char* e = getenv("NF4_GEMM_TM")) {     // tuning override
        const int v = atoi(e);
        if ((v == 32 || v == 64 || v == 128 || v == 256) && v <= TM) TM = v;
    }
    const int64_t ctas = ((N + GM_BM - 1) / GM_BM) * ((M + TM - 1) / TM);
    int64_t splits = GM_SM_TARGET / ctas;            // one CTA per SM is resident
    const int64_t KB = K / 64;
    const int64_t max_splits = KB % GM_WKB == 0 ? KB / GM_WKB : KB;    // ranges are whole groups when they can be
    // a range keeps at least 4 K blocks; 48 for tall tiles, whose fp32 partial sums (TM x 128 x 4 bytes per
    // split) cost as much as dozens of K blocks (measured: 4096x4096, M=256 loses 40 % with 16-block ranges,
    // 4096x14336 gains 50 % with 56-block ranges)
    const int64_t min_kb = TM > 64 ? 48 : 4;
    if (splits > KB / min_kb) splits = KB / min_kb;
    if (splits < 1) splits = 1;
    const char* e = getenv("NF4_GEMM_SPLITS");
    const int forced = e ? atoi(e) : -1;
    if (forced >= 1) splits = forced;
    if (splits > max_splits) splits = max_splits;
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
    const int v = e ? atoi(e) : 17;     // up to 16 rows the fused GEMV is faster on every shape measured
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
    // two CTAs per tile pair (see the head of this file): tall tiles, no K split, weight tiles in pairs.  Correct
    // but measured 3-10 % slower than one CTA per tile on every shape tried, so it runs only when asked for
    bool pair = false;
    if (const char* e = getenv("NF4_GEMM_PAIR")) {
        pair = atoi(e) == 1 && TM == 256 && splits == 1 && ntiles % 2 == 0 && ex.epilogue == 0;
    }
    const int smem_bytes = gemm_layout(TM, pair, &p);
    p.absmax = absmax; p.code16 = code16; p.bias = bias; p.y = y;
    p.residual = ex.residual; p.epilogue = ex.epilogue; p.pdl = ex.pdl;
    p.counters = static_cast<unsigned*>(ex.workspace);
    p.partials = ex.workspace ? reinterpret_cast<float*>(static_cast<uint8_t*>(ex.workspace) + GM_COUNTER_BYTES) : nullptr;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.KB = (int)(K / 64);
    p.am_tma = (p.KB % GM_WKB == 0 && reinterpret_cast<uintptr_t>(absmax) % 16 == 0) ? 1 : 0;
    const cuuint32_t estr[2] = {1, 1};
    if (p.am_tma) {
        const cuuint64_t dim[2] = {(cuuint64_t)p.KB, (cuuint64_t)N};
        const cuuint64_t str[1] = {(cuuint64_t)p.KB * 4};
        const cuuint32_t box[2] = {(cuuint32_t)GM_WKB, (cuuint32_t)GM_BM};
        CUresult r = enc(&p.amap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(absmax), dim, str, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        NF4_REQUIRE(r == CUDA_SUCCESS, NF4_ERR_CUDA, "gemm: cuTensorMapEncodeTiled(absmax) failed with %d", (int)r);
    } else {
        memset(&p.amap, 0, sizeof(p.amap));
    }
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
        const cuuint32_t box[2] = {64, (cuuint32_t)(pair ? TM / 2 : TM)};
        CUresult r = enc(&p.xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dim, str, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        NF4_REQUIRE(r == CUDA_SUCCESS, NF4_ERR_CUDA, "gemm: cuTensorMapEncodeTiled(activations) failed with %d", (int)r);
    }
    static bool configured[64] = {false};
    int dev = 0;
    NF4_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        NF4_CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
        NF4_CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
        configured[dev] = true;
    }
    dim3 grid((unsigned)ntiles, (unsigned)(mtiles * splits));
    NF4_REQUIRE(grid.y <= 65535, NF4_ERR_LIMIT, "gemm: M=%lld too large", (long long)M);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(GM_THREADS);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int nattr = 0;
    if (ex.pdl) {
        attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[nattr].val.programmaticStreamSerializationAllowed = 1;
        ++nattr;
    }
    if (pair) {
        attr[nattr].id = cudaLaunchAttributeClusterDimension;
        attr[nattr].val.clusterDim.x = 2;
        attr[nattr].val.clusterDim.y = 1;
        attr[nattr].val.clusterDim.z = 1;
        ++nattr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
    if (pair) NF4_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<true>, p));
    else NF4_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<false>, p));
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
