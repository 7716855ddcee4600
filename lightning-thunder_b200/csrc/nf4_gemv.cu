// Fused NF4 dequant-GEMV for the decode regime (M <= 16 activation rows), sm_100a.
//
//   y[m][n] = sum_k x[m][k] * code16[idx[n][k]] * absmax[n][k/64]  (+ bias[n])
//
// HBM-bound: every packed byte and absmax value is read exactly once.  Algorithmic bytes per
// call: N*K/2 (codes) + N*K/16 (absmax) + 2*M*K (x) + 2*M*N (y).
//
// Mapping (one persistent CTA of 16 warps per SM, each CTA owns a contiguous range of rows):
//  * weights are the A operand of mma.sync.m16n8k16 (16 weight rows x 16 k), the <= 8 activation
//    rows are the 8 columns of the B operand, so the same instruction stream serves M = 1..8 (two
//    column tiles for M = 9..16) and the multiply-adds run on the tensor pipe instead of 2 FMA
//    per weight on the fp32 pipe;
//  * a quad of threads loads the 32 packed bytes of one 64-element block of one row (8 bytes per
//    thread, straight from HBM into registers, L1 bypassed), so the 4 MMAs built from those bytes
//    stay inside one quantization block and the block's fp32 absmax is applied once to the 4
//    accumulators (acc += partial * absmax) instead of once per weight;
//  * nibble pairs are expanded by a 256-entry byte -> (bf16,bf16) table in shared memory,
//    replicated once per lane (entry stride 256 B, lane slot 4 B) so that a lookup never has a
//    bank conflict; the table window is 64 KB aligned, which lets ONE prmt build the complete
//    shared address (byte -> bits 8..15, lane slot and window base from the second operand);
//  * K is split over P warps of the CTA (each walks its own range of 64-blocks), partial sums
//    meet in shared memory once per batch of rows and the sum is written as bf16/fp16.
//    Summation order is fixed, so results are reproducible run to run.
#include <cstdio>
#include <cstdlib>

#include "nf4_gemv_common.cuh"

namespace nf4 {

constexpr int GEMV_THREADS = 512;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr int GEMV_NSTAGE = 3;             // register stages of weight loads (NSTAGE-1 in flight)
constexpr int X_SMEM_LIMIT = 60000;        // x is staged in shared memory when it fits below the table

struct GemvParams {
    const void* x;
    const uint8_t* packed;
    const float* absmax;
    const float* code16;
    const void* bias;
    const void* residual;   // optional [M][N], added after the bias (may alias y)
    void* y;
    int M, N, K;
    int KB;        // K / 64
    int log2P;     // warps along K
    int KBW;       // 64-blocks per warp = KB >> log2P
    int x_stride_bytes;  // row stride of the staged x in shared memory
};

template <int TB>
struct GemvStage {
    uint2 w[TB][2];    // packed bytes of rows (g, g+8) of TB row tiles, one 64-block
    float am[TB][2];
};

template <typename T, int NT, int TB, bool XSMEM>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int g = lane >> 2;   // row inside the tile / activation row
    const int q = lane & 3;

    const uint32_t s0 = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t lut_base = (s0 + LUT_WINDOW - 1) & ~(uint32_t)(LUT_WINDOW - 1);
    uint8_t* const lut_ptr = smem + (lut_base - s0);
    float* const part = reinterpret_cast<float*>(lut_ptr + LUT_WINDOW);
    const uint8_t* const xs = smem;   // staged activations (XSMEM)

    constexpr int PROWS = TB * 16;          // rows one warp produces per batch
    constexpr int PSTRIDE = PROWS + 4;      // padded so the 32 lanes of a store hit 32 banks
    constexpr int MCOLS = 8 * NT;
    constexpr int PART_FLOATS = GEMV_WARPS * MCOLS * PSTRIDE;   // one buffer

    const int P = 1 << p.log2P;
    const int R = GEMV_WARPS >> p.log2P;
    const int sg = warp & (P - 1);
    const int rg = warp >> p.log2P;

    // contiguous row range of this CTA
    const int r0 = (int)(((int64_t)p.N * blockIdx.x) / gridDim.x);
    const int r1 = (int)(((int64_t)p.N * (blockIdx.x + 1)) / gridDim.x);
    const int batch_rows = R * PROWS;
    const int nbatches = (r1 - r0 + batch_rows - 1) / batch_rows;
    const int nIter = nbatches * p.KBW;
    const int kb0 = sg * p.KBW;
    const int64_t row_bytes = (int64_t)p.K >> 1;

    GemvStage<TB> st[GEMV_NSTAGE];

    auto issue = [&](GemvStage<TB>& s, int it) {
        const int batch = it / p.KBW;
        const int kb = kb0 + (it - batch * p.KBW);
        const int rowbase = r0 + (batch * R + rg) * PROWS + g;
#pragma unroll
        for (int j = 0; j < TB; ++j) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = rowbase + j * 16 + h * 8;
                if (it < nIter && row < r1) {
                    s.w[j][h] = ld_nc_u64(p.packed + (int64_t)row * row_bytes + kb * 32 + q * 8);
                    s.am[j][h] = __ldg(p.absmax + (int64_t)row * p.KB + kb);
                } else {
                    s.w[j][h] = make_uint2(0u, 0u);
                    s.am[j][h] = 0.0f;
                }
            }
        }
    };

    // first loads go out before the table exists: HBM latency overlaps the set-up below
#pragma unroll
    for (int s = 0; s < GEMV_NSTAGE - 1; ++s) issue(st[s], s);

    // ---- set-up: lookup table, staged activations ------------------------------------------
    {
        const int slot = tid & 31;
#pragma unroll
        for (int i = 0; i < 256 / GEMV_WARPS; ++i) {
            const int e = warp + i * GEMV_WARPS;
            const uint32_t v = Mma<T>::pack(__ldg(p.code16 + (e >> 4)), __ldg(p.code16 + (e & 15)));
            *reinterpret_cast<uint32_t*>(lut_ptr + e * 256 + slot * 4) = v;
        }
        if constexpr (XSMEM) {
            const int chunks_per_row = p.K >> 3;   // 16-byte chunks
            const int total = p.M * chunks_per_row;
            for (int c = tid; c < total; c += GEMV_THREADS) {
                const int m = c / chunks_per_row;
                const int cc = c - m * chunks_per_row;
                const uint4 v = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.x) + ((int64_t)m * p.K << 1) + (cc << 4));
                *reinterpret_cast<uint4*>(const_cast<uint8_t*>(xs) + m * p.x_stride_bytes + (cc << 4)) = v;
            }
        }
    }
    __syncthreads();

    const uint32_t window_lane = lut_base | (uint32_t)(lane << 2);

    float acc[TB][NT][4];
#pragma unroll
    for (int j = 0; j < TB; ++j)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[j][nt][e] = 0.0f;

    const float zero4[4] = {0.0f, 0.0f, 0.0f, 0.0f};

    auto compute = [&](const GemvStage<TB>& s, int it) {
        const int batch = it / p.KBW;
        const int kbi = it - batch * p.KBW;
        const int kb = kb0 + kbi;

        // B fragments: 16 consecutive activations of row m = g (+8), k = kb*64 + 16q ..
        uint32_t xf[NT][8];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int m = g + nt * 8;
            if (m < p.M) {
                uint4 v0, v1;
                if constexpr (XSMEM) {
                    const uint4* src = reinterpret_cast<const uint4*>(xs + m * p.x_stride_bytes + ((kb * 64 + q * 16) << 1));
                    v0 = src[0];
                    v1 = src[1];
                } else {
                    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.x) +
                                                                      (((int64_t)m * p.K + kb * 64 + q * 16) << 1));
                    v0 = __ldg(src);
                    v1 = __ldg(src + 1);
                }
                xf[nt][0] = v0.x; xf[nt][1] = v0.y; xf[nt][2] = v0.z; xf[nt][3] = v0.w;
                xf[nt][4] = v1.x; xf[nt][5] = v1.y; xf[nt][6] = v1.z; xf[nt][7] = v1.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) xf[nt][i] = 0u;
            }
        }

#pragma unroll
        for (int j = 0; j < TB; ++j) {
            float tmp[NT][4];
            const uint32_t wa[2] = {s.w[j][0].x, s.w[j][0].y};
            const uint32_t wb[2] = {s.w[j][1].x, s.w[j][1].y};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                uint32_t a[4];
                const uint32_t va = wa[t >> 1], vb = wb[t >> 1];
                if (t & 1) {
                    a[0] = lut_lookup<2>(va, window_lane);
                    a[1] = lut_lookup<2>(vb, window_lane);
                    a[2] = lut_lookup<3>(va, window_lane);
                    a[3] = lut_lookup<3>(vb, window_lane);
                } else {
                    a[0] = lut_lookup<0>(va, window_lane);
                    a[1] = lut_lookup<0>(vb, window_lane);
                    a[2] = lut_lookup<1>(va, window_lane);
                    a[3] = lut_lookup<1>(vb, window_lane);
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    if (t == 0) Mma<T>::run(tmp[nt], a, xf[nt][0], xf[nt][1], zero4);
                    else Mma<T>::run(tmp[nt], a, xf[nt][2 * t], xf[nt][2 * t + 1], tmp[nt]);
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                acc[j][nt][0] = fmaf(tmp[nt][0], s.am[j][0], acc[j][nt][0]);
                acc[j][nt][1] = fmaf(tmp[nt][1], s.am[j][0], acc[j][nt][1]);
                acc[j][nt][2] = fmaf(tmp[nt][2], s.am[j][1], acc[j][nt][2]);
                acc[j][nt][3] = fmaf(tmp[nt][3], s.am[j][1], acc[j][nt][3]);
            }
        }

        if (kbi == p.KBW - 1) {
            // ---- end of a batch: partial sums meet in shared memory ---------------------------
            float* const pb = part + (batch & 1) * PART_FLOATS;
            float* const mine = pb + warp * (MCOLS * PSTRIDE);
#pragma unroll
            for (int j = 0; j < TB; ++j)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int m = nt * 8 + 2 * q;
                    if (m < p.M) {
                        mine[m * PSTRIDE + j * 16 + g] = acc[j][nt][0];
                        mine[m * PSTRIDE + j * 16 + g + 8] = acc[j][nt][2];
                    }
                    if (m + 1 < p.M) {
                        mine[(m + 1) * PSTRIDE + j * 16 + g] = acc[j][nt][1];
                        mine[(m + 1) * PSTRIDE + j * 16 + g + 8] = acc[j][nt][3];
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[j][nt][e] = 0.0f;
                }
            __syncthreads();
            const int outputs = p.M * batch_rows;
            for (int o = tid; o < outputs; o += GEMV_THREADS) {
                const int m = o / batch_rows;
                const int rr = o - m * batch_rows;      // rgi * PROWS + row
                const int rgi = rr / PROWS;
                const int row = rr - rgi * PROWS;
                const int grow = r0 + batch * batch_rows + rr;
                if (grow < r1) {
                    const float* src = pb + (rgi * P) * (MCOLS * PSTRIDE) + m * PSTRIDE + row;
                    float sum = 0.0f;
                    for (int k = 0; k < P; ++k) sum += src[k * (MCOLS * PSTRIDE)];
                    if (p.bias) sum += Elem<T>::to_f32(static_cast<const T*>(p.bias)[grow]);
                    if (p.residual) sum += Elem<T>::to_f32(static_cast<const T*>(p.residual)[(int64_t)m * p.N + grow]);
                    static_cast<T*>(p.y)[(int64_t)m * p.N + grow] = Elem<T>::from_f32(sum);
                }
            }
        }
    };

    for (int it = 0; it < nIter; it += GEMV_NSTAGE) {
#pragma unroll
        for (int s = 0; s < GEMV_NSTAGE; ++s) {
            if (it + s < nIter) {
                issue(st[(s + GEMV_NSTAGE - 1) % GEMV_NSTAGE], it + s + GEMV_NSTAGE - 1);
                compute(st[s], it + s);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Generic kernel: any K, any blocksize, fp32/fp16/bf16.  One warp per weight row, up to 16
// activation rows per pass.  Slow path for shapes the tensor-core kernels do not take.  Same
// numerics as the fused GEMV: levels rounded to the activation type, fp32 scaling and sums.
template <typename T>
__global__ void __launch_bounds__(256) linear_generic_kernel(const T* __restrict__ x, int M, int K,
                                                             const uint8_t* __restrict__ packed,
                                                             const float* __restrict__ absmax,
                                                             const float* __restrict__ code16, int N, int blocksize,
                                                             const T* __restrict__ bias, T* __restrict__ y) {
    __shared__ float s_code[16];
    if (threadIdx.x < 16) s_code[threadIdx.x] = Elem<T>::to_f32(Elem<T>::from_f32(code16[threadIdx.x]));
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= N) return;
    const int m0 = blockIdx.y * 16;
    const int mc = (M - m0) < 16 ? (M - m0) : 16;
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
    for (int k = lane; k < K; k += 32) {
        const int64_t i = n * K + k;
        const uint8_t byte = packed[i >> 1];
        const int idx = (i & 1) ? (byte & 15) : (byte >> 4);
        const float w = __fmul_rn(s_code[idx], absmax[i / blocksize]);
#pragma unroll
        for (int m = 0; m < 16; ++m)
            if (m < mc) acc[m] = fmaf(Elem<T>::to_f32(x[(int64_t)(m0 + m) * K + k]), w, acc[m]);
    }
#pragma unroll
    for (int m = 0; m < 16; ++m) {
        float v = acc[m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && m < mc) {
            if (bias) v += Elem<T>::to_f32(bias[n]);
            y[(int64_t)(m0 + m) * N + n] = Elem<T>::from_f32(v);
        }
    }
}

// ---------------------------------------------------------------------------------------------

struct GemvPlan { int TB, log2P, grid; bool xsmem; };

static GemvPlan plan_gemv(int M, int N, int K, int NT) {
    GemvPlan pl;
    const int sms = sm_count();
    const int KB = K / 64;
    int grid = sms;
    if (grid > (N + 15) / 16) grid = (N + 15) / 16;
    if (grid < 1) grid = 1;
    const int rho = (N + grid - 1) / grid;   // rows per CTA
    int maxlog2P = 0;
    while (maxlog2P < 4 && (KB % (2 << maxlog2P)) == 0) ++maxlog2P;
    // cost model: issued row-slots (masked rows still cost issue slots), the per-block activation
    // fetch shared by TB tiles, and a fixed price per batch (barrier + partial-sum exchange)
    double best = 1e30;
    pl.TB = 1; pl.log2P = maxlog2P;
    const int tb_max = NT == 1 ? 4 : 2;
    for (int TB = 1; TB <= tb_max; TB *= 2) {
        for (int lp = 0; lp <= maxlog2P; ++lp) {
            const int R = GEMV_WARPS >> lp;
            const int batch_rows = R * TB * 16;
            const int nb = (rho + batch_rows - 1) / batch_rows;
            const int KBW = KB >> lp;
            const double per_iter = TB * 1.0 + 0.25 * NT + 0.15;      // lookups + x fragment + loop overhead
            const double cost = nb * (KBW * per_iter + 6.0 + 0.5 * (1 << lp));
            if (cost < best) { best = cost; pl.TB = TB; pl.log2P = lp; }
        }
    }
    if (const char* env = getenv("NF4_GEMV_PLAN")) {   // "TB,log2P" override for tuning runs
        int tb = 0, lp = 0;
        if (sscanf(env, "%d,%d", &tb, &lp) == 2 && (tb == 1 || tb == 2 || (tb == 4 && NT == 1)) && lp >= 0 && lp <= maxlog2P) {
            pl.TB = tb; pl.log2P = lp;
        }
    }
    pl.grid = grid;
    pl.xsmem = (int64_t)M * (2 * (int64_t)K + 16) <= X_SMEM_LIMIT;
    return pl;
}

template <typename T, int NT, int TB, bool XS>
static int launch_gemv(const GemvParams& p, int grid, cudaStream_t stream) {
    static bool configured[64] = {false};
    int dev = 0;
    NF4_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        NF4_CUDA_TRY(cudaFuncSetAttribute(gemv_kernel<T, NT, TB, XS>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMV_SMEM));
        configured[dev] = true;
    }
    gemv_kernel<T, NT, TB, XS><<<grid, GEMV_THREADS, GEMV_SMEM, stream>>>(p);
    NF4_CUDA_TRY(cudaGetLastError());
    return NF4_OK;
}

template <typename T, int NT>
static int dispatch_gemv(const GemvParams& p, const GemvPlan& pl, cudaStream_t stream) {
    if (pl.xsmem) {
        switch (pl.TB) {
            case 1: return launch_gemv<T, NT, 1, true>(p, pl.grid, stream);
            case 2: return launch_gemv<T, NT, 2, true>(p, pl.grid, stream);
            case 4: if constexpr (NT == 1) return launch_gemv<T, NT, 4, true>(p, pl.grid, stream);
        }
    } else {
        switch (pl.TB) {
            case 1: return launch_gemv<T, NT, 1, false>(p, pl.grid, stream);
            case 2: return launch_gemv<T, NT, 2, false>(p, pl.grid, stream);
            case 4: if constexpr (NT == 1) return launch_gemv<T, NT, 4, false>(p, pl.grid, stream);
        }
    }
    set_error("gemv: no kernel for TB=%d NT=%d", pl.TB, NT);
    return NF4_ERR_ARG;
}

template <typename T>
static int gemv_typed(const void* x, int M, int K, const uint8_t* packed, const float* absmax, const float* code16,
                      int N, const void* bias, const void* residual, void* y, cudaStream_t stream,
                      const GemvOptions& opt = GemvOptions()) {
    const char* force = getenv("NF4_GEMV_KERNEL");   // "direct" or "staged": pins the variant (tests, tuning)
    if (opt.prologue != 0 || opt.epilogue != 0 || !(force && force[0] == 'd')) {
        const int rc = gemv_staged_try<T>(x, M, K, packed, absmax, code16, N, bias, residual, y, stream, opt);
        if (rc >= 0) return rc;
        if (opt.prologue != 0 || opt.epilogue != 0) {
            set_error("gemv: the fused prologue/epilogue needs M*K small enough to stage the activations (M=%d K=%d) and K a multiple of 256", M, K);
            return NF4_ERR_LIMIT;
        }
        if (force && force[0] == 's') {
            set_error("gemv: the staged kernel does not take M=%d N=%d K=%d", M, N, K);
            return NF4_ERR_ARG;
        }
    }
    const int NT = M <= 8 ? 1 : 2;
    GemvPlan pl = plan_gemv(M, N, K, NT);
    GemvParams p;
    p.x = x; p.packed = packed; p.absmax = absmax; p.code16 = code16; p.bias = bias; p.residual = residual; p.y = y;
    p.M = M; p.N = N; p.K = K; p.KB = K / 64; p.log2P = pl.log2P; p.KBW = p.KB >> pl.log2P;
    p.x_stride_bytes = 2 * K + 16;
    return NT == 1 ? dispatch_gemv<T, 1>(p, pl, stream) : dispatch_gemv<T, 2>(p, pl, stream);
}

bool gemv_supported(int64_t M, int64_t K, int64_t N, int blocksize, int dtype, const void* x, const void* packed,
                    const void* absmax) {
    return M >= 1 && M <= 16 && N >= 1 && K >= 64 && K % 64 == 0 && blocksize == 64 &&
           (dtype == NF4_BF16 || dtype == NF4_F16) && N * K < ((int64_t)1 << 40) && N < (1 << 30) && K < (1 << 24) &&
           reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(packed) % 8 == 0 &&
           reinterpret_cast<uintptr_t>(absmax) % 4 == 0;
}

}  // namespace nf4

using namespace nf4;

extern "C" int nf4_b200_gemv_fused(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                                   const float* code16, int64_t N, const void* bias, const void* residual, void* y,
                                   int dtype, void* stream) {
    NF4_REQUIRE(x && packed && absmax && code16 && y, NF4_ERR_ARG, "gemv: null pointer");
    NF4_REQUIRE(M >= 1 && M <= 16, NF4_ERR_ARG, "gemv: M=%lld outside [1,16]", (long long)M);
    NF4_REQUIRE(K >= 64 && K % 64 == 0, NF4_ERR_ARG, "gemv: K=%lld must be a positive multiple of 64", (long long)K);
    NF4_REQUIRE(N >= 1, NF4_ERR_ARG, "gemv: N=%lld < 1", (long long)N);
    NF4_REQUIRE(dtype == NF4_BF16 || dtype == NF4_F16, NF4_ERR_ARG, "gemv: dtype code %d is not fp16/bf16", dtype);
    NF4_REQUIRE(gemv_supported(M, K, N, 64, dtype, x, packed, absmax), NF4_ERR_ALIGN,
                "gemv: x must be 16-byte aligned, packed 8-byte aligned, extents below 2^30 x 2^24");
    if (int rc = check_device()) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == NF4_BF16)
        return gemv_typed<__nv_bfloat16>(x, (int)M, (int)K, packed, absmax, code16, (int)N, bias, residual, y, s);
    return gemv_typed<__half>(x, (int)M, (int)K, packed, absmax, code16, (int)N, bias, residual, y, s);
}

// hint for the next nf4_b200_gemv_decode call of this thread (consumed by it)
static thread_local const uint8_t* t_next_packed = nullptr;
static thread_local const float* t_next_absmax = nullptr;
static thread_local int64_t t_next_N = 0, t_next_K = 0;

extern "C" int nf4_b200_gemv_decode_next_weight(const uint8_t* packed, const float* absmax, int64_t N, int64_t K) {
    NF4_REQUIRE((packed && absmax && N >= 1 && K >= 64 && K % 64 == 0 && N < (1ll << 30) && K < (1ll << 24)) || (!packed && !absmax),
                NF4_ERR_ARG, "gemv_decode_next_weight: bad hint N=%lld K=%lld", (long long)N, (long long)K);
    t_next_packed = packed; t_next_absmax = absmax; t_next_N = N; t_next_K = K;
    return NF4_OK;
}

extern "C" int nf4_b200_gemv_decode(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                                    const float* code16, int64_t N, const void* residual, void* y, int prologue,
                                    const void* norm_w, float eps, int epilogue, int flags, void* stream) {
    NF4_REQUIRE(x && packed && absmax && code16 && y, NF4_ERR_ARG, "gemv_decode: null pointer");
    NF4_REQUIRE(M >= 1 && M <= 16, NF4_ERR_ARG, "gemv_decode: M=%lld outside [1,16]", (long long)M);
    NF4_REQUIRE(K >= 64 && K % 64 == 0 && N >= 1, NF4_ERR_ARG, "gemv_decode: bad extents N=%lld K=%lld", (long long)N, (long long)K);
    NF4_REQUIRE(prologue >= 0 && prologue <= 2, NF4_ERR_ARG, "gemv_decode: prologue %d", prologue);
    NF4_REQUIRE(prologue != 1 || norm_w, NF4_ERR_ARG, "gemv_decode: the rmsnorm prologue needs norm_w");
    NF4_REQUIRE(epilogue == 0 || (epilogue == 1 && !residual && N % 2 == 0) || (epilogue == 2 && !residual && N % 16 == 0),
                NF4_ERR_ARG, "gemv_decode: the SwiGLU epilogues take no residual and an even N (pairs) or N %% 16 == 0 (halves)");
    NF4_REQUIRE(gemv_supported(M, K, N, 64, NF4_BF16, x, packed, absmax), NF4_ERR_ALIGN,
                "gemv_decode: x must be 16-byte aligned, packed 8-byte aligned");
    if (int rc = check_device()) return rc;
    GemvOptions opt;
    opt.prologue = prologue; opt.norm_w = norm_w; opt.eps = eps; opt.epilogue = epilogue; opt.pdl = (flags & 1) != 0;
    opt.next_packed = t_next_packed; opt.next_absmax = t_next_absmax; opt.next_N = (int)t_next_N; opt.next_K = (int)t_next_K;
    t_next_packed = nullptr; t_next_absmax = nullptr;
    return gemv_typed<__nv_bfloat16>(x, (int)M, (int)K, packed, absmax, code16, (int)N, nullptr, residual, y,
                                     static_cast<cudaStream_t>(stream), opt);
}

// Fused GEMV on a double-quantized weight: the uint8 absmax indices are expanded inside the kernel's stages.
// Returns -1 (nothing launched) when the shape or a pointer does not suit that kernel.
namespace nf4 {
int gemv_dq_try(const void* x, int64_t M, int64_t K, const uint8_t* packed, const uint8_t* absmax_u8, const float* scale2,
                const float* offset, const float* code256, const float* code16, int64_t N, const void* bias, void* y,
                int dtype, cudaStream_t stream) {
    if (dtype != NF4_BF16 || M < 1 || M > 16 || K < 64 || K % 64 != 0 || N < 1) return -1;
    if (!gemv_supported(M, K, N, 64, dtype, x, packed, code16)) return -1;
    GemvOptions opt;
    opt.dq_absmax_u8 = absmax_u8; opt.dq_scale2 = scale2; opt.dq_offset = offset; opt.dq_code256 = code256;
    const int rc = gemv_staged_try<__nv_bfloat16>(x, (int)M, (int)K, packed, nullptr, code16, (int)N, bias, nullptr, y, stream, opt);
    return rc < 0 ? -1 : rc;
}
}  // namespace nf4

extern "C" int nf4_b200_gemv(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                             const float* code16, int64_t N, const void* bias, void* y, int dtype, void* stream) {
    return nf4_b200_gemv_fused(x, M, K, packed, absmax, code16, N, bias, nullptr, y, dtype, stream);
}

extern "C" int nf4_b200_linear_generic(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                                       const float* code16, int64_t N, int blocksize, const void* bias, void* y,
                                       int dtype, void* stream) {
    NF4_REQUIRE(M >= 0 && N >= 0 && K >= 0, NF4_ERR_ARG, "linear_generic: negative extent");
    NF4_REQUIRE(blocksize >= 2 && (blocksize & 1) == 0, NF4_ERR_ARG, "linear_generic: blocksize %d", blocksize);
    if (M == 0 || N == 0) return NF4_OK;
    NF4_REQUIRE(x && packed && absmax && code16 && y, NF4_ERR_ARG, "linear_generic: null pointer");
    NF4_REQUIRE(M < (1 << 30) && N < (1 << 30) && K < (1 << 30), NF4_ERR_LIMIT, "linear_generic: extent above 2^30");
    if (int rc = check_device()) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int warps = 8;
    dim3 grid((unsigned)((N + warps - 1) / warps), (unsigned)((M + 15) / 16));
    NF4_REQUIRE(grid.y <= 65535, NF4_ERR_LIMIT, "linear_generic: M=%lld too large for this kernel", (long long)M);
    switch (dtype) {
        case NF4_F32:
            linear_generic_kernel<float><<<grid, warps * 32, 0, s>>>(static_cast<const float*>(x), (int)M, (int)K, packed, absmax, code16,
                                                                      (int)N, blocksize, static_cast<const float*>(bias), static_cast<float*>(y));
            break;
        case NF4_F16:
            linear_generic_kernel<__half><<<grid, warps * 32, 0, s>>>(static_cast<const __half*>(x), (int)M, (int)K, packed, absmax, code16,
                                                                       (int)N, blocksize, static_cast<const __half*>(bias), static_cast<__half*>(y));
            break;
        case NF4_BF16:
            linear_generic_kernel<__nv_bfloat16><<<grid, warps * 32, 0, s>>>(static_cast<const __nv_bfloat16*>(x), (int)M, (int)K, packed, absmax,
                                                                              code16, (int)N, blocksize, static_cast<const __nv_bfloat16*>(bias),
                                                                              static_cast<__nv_bfloat16*>(y));
            break;
        default:
            set_error("linear_generic: unknown dtype code %d", dtype);
            return NF4_ERR_ARG;
    }
    NF4_CUDA_TRY(cudaGetLastError());
    return NF4_OK;
}
