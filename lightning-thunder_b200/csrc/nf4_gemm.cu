// Prefill-regime NF4 dequant-GEMM (M > 16) on the 5th-generation tensor cores (tcgen05 / TMEM).
//
//   y[m][n] = sum_k x[m][k] * W[n][k] + bias[n],   W[n][k] = bf16( bf16(code[idx]) * absmax[n][k/64] )
//
// One CTA computes a tile of 128 weight rows x TM (<= 256) activation rows; weights are the A operand
// (UMMA M = 128), activations the B operand (UMMA N = TM), both K-major bf16 in shared memory with
// the 128-byte swizzle, the fp32 accumulator lives in TMEM (TM columns).  Per 64-element K block
// (= one quantization block per row, one 128-byte swizzle atom):
//   warp 0   (producer)  TMA: box of 128 rows x 32 packed bytes (+16 bytes of padding per row so the
//                        row pitch of 48 B keeps 16-byte reads of 8 consecutive rows conflict-free)
//                        and box of TM x 64 activations (SWIZZLE_128B) -> mbarrier `full`
//   warps 2-9 (dequant)  two threads per weight row, 16 bytes -> 32 bf16 each, through the byte->(bf16,bf16)
//                        table, scaled by the row's fp32 absmax in fp32, rounded once, stored as
//                        8 x 16-byte chunks at the swizzled positions of the A stage; then
//                        fence.proxy.async + arrive on `a_ready`
//   warp 1   (MMA)       one elected thread issues 4 x tcgen05.mma (K = 16 each) per block and commits
//                        to `empty` (frees the stage) -- after the last block to `acc_done`
// Epilogue (warps 2-5): tcgen05.ld 32 lanes x 32 columns at a time, + bias, bf16, store to y[m][n]
// (a warp writes 32 consecutive n for one m: 64-byte segments).
//
// Every mbarrier wait is bounded; a time-out sets a status word (nf4_b200_device_error code 5..8),
// the CTA stops waiting and runs to its end (TMEM is always released).
#include <cuda.h>

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
constexpr int GM_THREADS = (2 + GM_DQ_WARPS) * 32;   // producer, MMA, dequant (the first 4 also run the epilogue)
constexpr int GM_BM = 128;               // weight rows per CTA (UMMA M)
constexpr int GM_STAGES = 3;
constexpr int GM_PK_PITCH = 48;          // bytes per row of a packed stage (32 used)
constexpr int GM_A_BYTES = GM_BM * 128;  // 128 rows x 64 bf16
constexpr int GM_PK_BYTES = GM_BM * GM_PK_PITCH;
constexpr int GM_LUT_BYTES = 256 * 128;  // byte -> (bf16,bf16), one copy per lane
constexpr unsigned long long GM_WAIT_LIMIT_NS = 200ull * 1000 * 1000;

struct alignas(64) GemmParams {
    CUtensorMap wmap;     // packed codes uint8 [N][K/2], box 48 x 128
    CUtensorMap xmap;     // activations bf16 [M][K], box 64 x TM, SWIZZLE_128B
    const float* absmax;
    const float* code16;
    const void* bias;
    void* y;
    int M, N, K, KB;
    int TM;               // activation rows per CTA: multiple of 16, 32..256
    int tmem_cols;        // power of two >= TM, >= 32
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
    uint8_t* const a_base = smem;                                      // GM_STAGES x 16 KB
    uint8_t* const b_base = a_base + GM_STAGES * GM_A_BYTES;           // GM_STAGES x TM*128
    uint8_t* const pk_base = b_base + GM_STAGES * b_bytes;             // GM_STAGES x 6 KB
    uint8_t* const lut = pk_base + GM_STAGES * GM_PK_BYTES;            // 32 KB
    uint64_t* const bars = reinterpret_cast<uint64_t*>(lut + GM_LUT_BYTES);
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* const abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t full0 = gm_smem_u32(bars), aready0 = full0 + 8 * GM_STAGES, empty0 = full0 + 16 * GM_STAGES,
                   accdone = full0 + 24 * GM_STAGES;

    const int n0 = blockIdx.x * GM_BM;
    const int m0 = blockIdx.y * TM;

    if (tid == 0) {
        for (int s = 0; s < GM_STAGES; ++s) {
            gm_mbar_init(full0 + 8 * s, 1);
            gm_mbar_init(aready0 + 8 * s, GM_DQ_WARPS);     // one arrival per dequant warp
            gm_mbar_init(empty0 + 8 * s, 1);      // tcgen05.commit
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
    if (warp >= 2) {
        // byte -> (bf16(code[hi]), bf16(code[lo])) table, one copy per lane (conflict-free lookups)
        for (int e = warp - 2; e < 256; e += GM_DQ_WARPS) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(__ldg(p.code16 + (e >> 4)), __ldg(p.code16 + (e & 15)));
            *reinterpret_cast<uint32_t*>(lut + e * 128 + lane * 4) = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;

    const int KB = p.KB;
    if (warp == 0) {
        // ------------------------------------ producer ----------------------------------------
        int slot = 0;
        uint32_t parity = 0;
        for (int kb = 0; kb < KB; ++kb) {
            gm_wait(empty0 + 8 * slot, parity ^ 1u, abort_flag, 6, kb);
            if (lane == 0) {
                const uint32_t fb = full0 + 8 * slot;
                gm_mbar_expect_tx(fb, (uint32_t)(GM_PK_BYTES + b_bytes));
                gm_tma_2d(gm_smem_u32(pk_base + slot * GM_PK_BYTES), &p.wmap, kb * 32, n0, fb);
                gm_tma_2d(gm_smem_u32(b_base + slot * b_bytes), &p.xmap, kb * 64, m0, fb);
            }
            __syncwarp();
            if (++slot == GM_STAGES) { slot = 0; parity ^= 1u; }
        }
    } else if (warp == 1) {
        // ------------------------------------ MMA issuer ---------------------------------------
        const uint32_t idesc = gm_instr_desc(TM);
        int slot = 0;
        uint32_t parity = 0;
        for (int kb = 0; kb < KB; ++kb) {
            gm_wait(full0 + 8 * slot, parity, abort_flag, 5, kb);      // activations landed
            gm_wait(aready0 + 8 * slot, parity, abort_flag, 7, kb);    // weights dequantised
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const uint64_t adesc = gm_smem_desc(gm_smem_u32(a_base + slot * GM_A_BYTES));
                const uint64_t bdesc = gm_smem_desc(gm_smem_u32(b_base + slot * b_bytes));
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                    // advancing 16 elements along K inside the swizzle atom = +32 bytes = +2 in the address field
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "setp.ne.u32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                        ::"r"(tmem_d), "l"(adesc + (uint64_t)(2 * k)), "l"(bdesc + (uint64_t)(2 * k)), "r"(idesc), "r"(accumulate)
                        : "memory");
                }
                // frees the stage once these MMAs have read it
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(empty0 + 8 * slot) : "memory");
                if (kb == KB - 1)
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(accdone) : "memory");
            }
            __syncwarp();
            if (++slot == GM_STAGES) { slot = 0; parity ^= 1u; }
        }
    } else {
        // ------------------------------------ dequant warps -------------------------------------
        const int t = tid - 64;                 // 0..255
        const int r = t & 127;                  // weight row inside the tile
        const int hsel = t >> 7;                // which half of the row's 64-block: bytes [16*hsel, 16*hsel+16)
        const int grow = n0 + r;
        const uint32_t lut_lane = gm_smem_u32(lut) + (uint32_t)lane * 4u;
        int slot = 0;
        uint32_t parity = 0;
        float am_next = grow < p.N ? __ldg(p.absmax + (int64_t)grow * KB) : 0.0f;
        for (int kb = 0; kb < KB; ++kb) {
            const float am = am_next;
            if (kb + 1 < KB) am_next = grow < p.N ? __ldg(p.absmax + (int64_t)grow * KB + kb + 1) : 0.0f;
            gm_wait(full0 + 8 * slot, parity, abort_flag, 5, kb);       // packed bytes landed
            gm_wait(empty0 + 8 * slot, parity ^ 1u, abort_flag, 6, kb); // the A stage is free
            const uint4 w4 = *reinterpret_cast<const uint4*>(pk_base + slot * GM_PK_BYTES + r * GM_PK_PITCH + hsel * 16);
            const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
            uint8_t* const arow = a_base + slot * GM_A_BYTES + r * 128;
#pragma unroll
            for (int c = 0; c < 4; ++c) {       // 16-byte chunk = 8 weights = 4 packed bytes = one word
                uint32_t out[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t byte = __byte_perm(words[c], 0u, 0x4440 | j);
                    uint32_t pair;
                    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(pair) : "r"(lut_lane + byte * 128u));
                    const float lo = __uint_as_float(pair << 16) * am;
                    const float hi = __uint_as_float(pair & 0xffff0000u) * am;
                    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                    out[j] = *reinterpret_cast<const uint32_t*>(&h);
                }
                const int chunk = hsel * 4 + c;
                *reinterpret_cast<uint4*>(arow + ((chunk ^ (r & 7)) << 4)) = make_uint4(out[0], out[1], out[2], out[3]);
            }
            // generic-proxy stores must be visible to the tensor core (async proxy)
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) gm_mbar_arrive(aready0 + 8 * slot);
            if (++slot == GM_STAGES) { slot = 0; parity ^= 1u; }
        }
        if (warp >= 6) goto done;               // the epilogue needs one warp per TMEM lane quarter
        // ------------------------------------ epilogue ------------------------------------------
        gm_wait(accdone, 0u, abort_flag, 8, KB);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;          // accumulator lane = weight row inside the tile
        const int gn = n0 + row;
        const float bias = (p.bias && gn < p.N) ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[gn]) : 0.0f;
        __nv_bfloat16* const y = static_cast<__nv_bfloat16*>(p.y);
        for (int c0 = 0; c0 < TM; c0 += 16) {
            uint32_t v[16];
            const uint32_t taddr = tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                  "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                : "r"(taddr) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (gn < p.N) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int m = m0 + c0 + j;
                    if (m < p.M) y[(int64_t)m * p.N + gn] = __float2bfloat16_rn(__uint_as_float(v[j]) + bias);
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
    return GM_STAGES * (GM_A_BYTES + TM * 128 + GM_PK_BYTES) + GM_LUT_BYTES + 256;
}

bool gemm_supported(int64_t M, int64_t K, int64_t N, int blocksize, int dtype, const void* x, const void* packed,
                    const void* absmax, const void* y) {
    (void)y;
    return M > 16 && dtype == NF4_BF16 && blocksize == 64 && K >= 64 && K % 64 == 0 && N >= 1 && M < (1ll << 30) &&
           N < (1ll << 30) && K < (1ll << 24) && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
           reinterpret_cast<uintptr_t>(packed) % 16 == 0 && reinterpret_cast<uintptr_t>(absmax) % 4 == 0;
}

static int gemm_tcgen05(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax, const float* code16,
                        int64_t N, const void* bias, void* y, cudaStream_t stream) {
    GmEncodeFn enc = gm_encode_fn();
    NF4_REQUIRE(enc, NF4_ERR_CUDA, "gemm: cuTensorMapEncodeTiled is not available from this driver");
    GemmParams p;
    int TM = 256;
    while (TM > 32 && TM / 2 >= M) TM /= 2;         // 32, 64, 128 or 256 activation rows per CTA
    p.TM = TM;
    p.tmem_cols = TM;                               // a power of two >= 32
    p.absmax = absmax; p.code16 = code16; p.bias = bias; p.y = y;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.KB = (int)(K / 64);
    const cuuint32_t estr[2] = {1, 1};
    {
        const cuuint64_t dim[2] = {(cuuint64_t)(K / 2), (cuuint64_t)N};
        const cuuint64_t str[1] = {(cuuint64_t)(K / 2)};
        const cuuint32_t box[2] = {(cuuint32_t)GM_PK_PITCH, (cuuint32_t)GM_BM};
        CUresult r = enc(&p.wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(packed), dim, str, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
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
    dim3 grid((unsigned)((N + GM_BM - 1) / GM_BM), (unsigned)((M + TM - 1) / TM));
    NF4_REQUIRE(grid.y <= 65535, NF4_ERR_LIMIT, "gemm: M=%lld too large", (long long)M);
    gemm_tcgen05_kernel<<<grid, GM_THREADS, gemm_smem_bytes(TM), stream>>>(p);
    NF4_CUDA_TRY(cudaGetLastError());
    return NF4_OK;
}

}  // namespace nf4

using namespace nf4;

extern "C" int nf4_b200_gemm(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                             const float* code16, int64_t N, const void* bias, void* y, int dtype, void* workspace,
                             int64_t workspace_bytes, void* stream) {
    (void)workspace; (void)workspace_bytes;
    NF4_REQUIRE(x && packed && absmax && code16 && y, NF4_ERR_ARG, "gemm: null pointer");
    NF4_REQUIRE(M >= 1 && N >= 1, NF4_ERR_ARG, "gemm: M=%lld N=%lld", (long long)M, (long long)N);
    NF4_REQUIRE(K >= 64 && K % 64 == 0, NF4_ERR_ARG, "gemm: K=%lld must be a positive multiple of 64", (long long)K);
    NF4_REQUIRE(dtype == NF4_BF16 || dtype == NF4_F16, NF4_ERR_ARG, "gemm: dtype code %d is not fp16/bf16", dtype);
    if (int rc = check_device()) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (gemm_supported(M > 16 ? M : 17, K, N, 64, dtype, x, packed, absmax, y))
        return gemm_tcgen05(x, M, K, packed, absmax, code16, N, bias, y, s);
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
