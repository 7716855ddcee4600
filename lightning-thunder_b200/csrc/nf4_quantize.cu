// NF4 blockwise quantize and dequantize kernels (HBM-bound streaming kernels).
//
// quantize: each thread owns 8 consecutive elements (one 16-byte load for 16-bit inputs), a group
// of blocksize/8 adjacent threads owns one quantization block, the block absmax is a shuffle (and,
// above 256 elements, shared-memory) max, every element is divided by it and mapped to its level
// by counting decision thresholds (see level_threshold), and the 8 indices leave as one 32-bit
// store.  Algorithmic traffic per element: sizeof(T) read + 1/2 + 4/blocksize bytes written.
//
// dequantize: the mirror image; 4 packed bytes in, 8 elements out per thread.
#include "nf4_common.cuh"

namespace nf4 {

constexpr int QTHREADS = 256;

// index(v) = number of thresholds <= v, as a 4-step binary search over 15 sorted thresholds
// held in shared memory (padded to 16 with +inf so every probe is in range).
__device__ __forceinline__ uint32_t nf4_index(float v, const float* thr /*[16], thr[15]=+inf*/) {
    uint32_t i = (v >= thr[7]) ? 8u : 0u;
    i += (v >= thr[i + 3]) ? 4u : 0u;
    i += (v >= thr[i + 1]) ? 2u : 0u;
    i += (v >= thr[i]) ? 1u : 0u;
    return i;
}

// Bucketed search.  bucket(v) = low bits of the fp32 sum v*16 + 16 + 2^23 (a monotone function of v
// with 33 values on [-1, 1]).  If every bucket holds at most one threshold -- true whenever adjacent
// thresholds are more than 1/16 apart, as for NF4 -- then
//     index(v) = #{thresholds in lower buckets} + (v >= the threshold of v's own bucket),
// which equals the threshold count exactly because bucket() is monotone.  tab[b] = (count, threshold).
struct BucketTable { float2 tab[33]; int ok; };

__device__ __forceinline__ int nf4_bucket(float v) {
    return __float_as_int(__fmaf_rn(v, 16.0f, 8388624.0f)) & 63;
}

// called by threads 0..32 after thr[0..14] are in shared memory (followed by a barrier)
__device__ __forceinline__ void bucket_table_build(BucketTable& bt, const float* thr, int tid) {
    if (tid == 0) bt.ok = 1;
    __syncthreads();
    if (tid < 33) {
        int below = 0, here = 0;
        float mine = __int_as_float(0x7f800000);
        for (int i = 0; i < 15; ++i) {
            const int b = nf4_bucket(thr[i]);
            if (b < tid) ++below;
            if (b == tid) { ++here; mine = thr[i]; }
        }
        bt.tab[tid] = make_float2(__int_as_float(below), mine);
        if (here > 1) bt.ok = 0;
    }
}

__device__ __forceinline__ uint32_t nf4_index_bucketed(float v, const BucketTable& bt) {
    const float2 e = bt.tab[nf4_bucket(v)];
    return (uint32_t)__float_as_int(e.x) + (v >= e.y ? 1u : 0u);
}

// 8 consecutive elements as they sit in memory (one 16-byte word for 16-bit types, two for fp32) and their
// widening to fp32; the quantize loop keeps loads in flight in this raw form (fewer registers than 8 floats)
template <typename T> struct Raw8 { uint4 a; };
template <> struct Raw8<float> { uint4 a, b; };

template <typename T>
__device__ __forceinline__ Raw8<T> load_raw8(const T* p) {
    Raw8<T> r;
    r.a = ld_nc_u128(p);
    if constexpr (sizeof(T) == 4) r.b = ld_nc_u128(p + 4);
    return r;
}
template <typename T>
__device__ __forceinline__ Raw8<T> zero_raw8() {
    Raw8<T> r;
    r.a = make_uint4(0u, 0u, 0u, 0u);
    if constexpr (sizeof(T) == 4) r.b = r.a;
    return r;
}
__device__ __forceinline__ void widen8(const Raw8<float>& r, float (&v)[8]) {
    v[0] = __uint_as_float(r.a.x); v[1] = __uint_as_float(r.a.y); v[2] = __uint_as_float(r.a.z); v[3] = __uint_as_float(r.a.w);
    v[4] = __uint_as_float(r.b.x); v[5] = __uint_as_float(r.b.y); v[6] = __uint_as_float(r.b.z); v[7] = __uint_as_float(r.b.w);
}
__device__ __forceinline__ void widen8(const Raw8<__nv_bfloat16>& r, float (&v)[8]) {
    const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void widen8(const Raw8<__half>& r, float (&v)[8]) {
    const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

// Fast path: numel8 groups of 8 elements, all quantization blocks complete, w 16-byte aligned.
// GROUP = blocksize / 8 threads share one absmax (GROUP is a power of two, 8..512; <= QTHREADS).
template <typename T, int GROUP>
__global__ void __launch_bounds__(QTHREADS) quantize_kernel(const T* __restrict__ w, int64_t ngroups8,
                                                            const float* __restrict__ code16,
                                                            uint32_t* __restrict__ packed32,
                                                            float* __restrict__ absmax) {
    __shared__ float s_thr[16];
    __shared__ float s_max[QTHREADS / 32];
    __shared__ BucketTable s_bt;
    if (threadIdx.x < 15) s_thr[threadIdx.x] = level_threshold(code16[threadIdx.x], code16[threadIdx.x + 1]);
    if (threadIdx.x == 15) s_thr[15] = __int_as_float(0x7f800000);
    __syncthreads();
    bucket_table_build(s_bt, s_thr, threadIdx.x);
    __syncthreads();
    const bool bucketed = s_bt.ok != 0;

    const int64_t stride = (int64_t)gridDim.x * QTHREADS;
    // all threads of a CTA iterate the same number of times (shared-memory max needs barriers)
    const int64_t niter = (ngroups8 + stride - 1) / stride;
    // the loads of the next QAHEAD iterations are in flight during this iteration's arithmetic (the kernel waits on
    // its loads: with one load ahead it ran at 0.375 of the copy bandwidth, with two at 0.42, with three -- 48
    // registers instead of 40 -- at 0.40)
    constexpr int QAHEAD = 2;
    const int64_t t00 = (int64_t)blockIdx.x * QTHREADS + threadIdx.x;
    Raw8<T> ahead[QAHEAD];
#pragma unroll
    for (int a = 0; a < QAHEAD; ++a)
        ahead[a] = t00 + a * stride < ngroups8 ? load_raw8<T>(w + (t00 + a * stride) * 8) : zero_raw8<T>();
    for (int64_t it = 0; it < niter; ++it) {
        const int64_t t = it * stride + t00;
        const bool live = t < ngroups8;
        float v[8];
        widen8(ahead[0], v);
#pragma unroll
        for (int a = 0; a + 1 < QAHEAD; ++a) ahead[a] = ahead[a + 1];
        ahead[QAHEAD - 1] = t + QAHEAD * stride < ngroups8 ? load_raw8<T>(w + (t + QAHEAD * stride) * 8) : zero_raw8<T>();
        float am = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) am = fmaxf(am, fabsf(v[i]));
        constexpr int SHFL = GROUP < 32 ? GROUP : 32;
#pragma unroll
        for (int o = SHFL / 2; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        if constexpr (GROUP > 32) {
            // GROUP/32 warps share a block; QTHREADS % GROUP == 0 keeps blocks inside the CTA
            constexpr int WPB = GROUP / 32;
            const int warp = threadIdx.x >> 5;
            __syncthreads();
            if ((threadIdx.x & 31) == 0) s_max[warp] = am;
            __syncthreads();
            const int w0 = warp & ~(WPB - 1);
            am = s_max[w0];
#pragma unroll
            for (int i = 1; i < WPB; ++i) am = fmaxf(am, s_max[w0 + i]);
        }
        if (live) {
            uint32_t word = 0;
            // An all-zero block divides by 1: every quotient is 0 and maps to the level nearest 0.
            // Scales outside [2^-100, 2^100] take the compiler's fully guarded division.
            const float dv = am == 0.0f ? 1.0f : am;
            const bool bounded = dv >= 7.8886e-31f && dv <= 1.2676e30f;
            // the two choices below are uniform per block / per CTA: they select one of three straight-line
            // loops instead of being re-decided for every element
            if (bounded && bucketed) {
                const float rcp = refined_rcp(dv);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t idx = nf4_index_bucketed(div_rn_bounded(v[i], dv, rcp), s_bt);
                    // element 2j -> high nibble of byte j; bytes are little-endian inside the word
                    word |= idx << ((i >> 1) * 8 + ((i & 1) ? 0 : 4));
                }
            } else if (bounded) {
                const float rcp = refined_rcp(dv);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    word |= nf4_index(div_rn_bounded(v[i], dv, rcp), s_thr) << ((i >> 1) * 8 + ((i & 1) ? 0 : 4));
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    word |= nf4_index(__fdiv_rn(v[i], dv), s_thr) << ((i >> 1) * 8 + ((i & 1) ? 0 : 4));
            }
            packed32[t] = word;
            if ((t & (GROUP - 1)) == 0) absmax[t / GROUP] = am;
        }
    }
}

// Any extent / alignment: one thread per quantization block.  Used for short tensors, the ragged
// tail block and unaligned inputs.
template <typename T>
__global__ void quantize_tail_kernel(const T* __restrict__ w, int64_t first_block, int64_t numel, int blocksize,
                                     const float* __restrict__ code16, uint8_t* __restrict__ packed,
                                     float* __restrict__ absmax) {
    __shared__ float s_thr[16];
    __shared__ int s_zero;
    if (threadIdx.x < 15) s_thr[threadIdx.x] = level_threshold(code16[threadIdx.x], code16[threadIdx.x + 1]);
    if (threadIdx.x == 15) s_thr[15] = __int_as_float(0x7f800000);
    if (threadIdx.x == 16) {
        int z = 0;
        for (int i = 0; i < 16; ++i) if (code16[i] == 0.0f) { z = i; break; }
        s_zero = z;
    }
    __syncthreads();
    const int64_t nblocks = (numel + blocksize - 1) / blocksize;
    for (int64_t b = first_block + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks;
         b += (int64_t)gridDim.x * blockDim.x) {
        const int64_t lo = b * blocksize;
        const int64_t hi = (lo + blocksize < numel) ? lo + blocksize : numel;
        float am = 0.0f;
        for (int64_t i = lo; i < hi; ++i) am = fmaxf(am, fabsf(Elem<T>::to_f32(w[i])));
        absmax[b] = am;
        for (int64_t i = lo; i < hi; i += 2) {   // lo is even (blocksize is even)
            uint32_t i0 = (am == 0.0f) ? (uint32_t)s_zero : nf4_index(__fdiv_rn(Elem<T>::to_f32(w[i]), am), s_thr);
            uint32_t i1 = 0;
            if (i + 1 < hi) i1 = (am == 0.0f) ? (uint32_t)s_zero : nf4_index(__fdiv_rn(Elem<T>::to_f32(w[i + 1]), am), s_thr);
            packed[i >> 1] = (uint8_t)((i0 << 4) | i1);
        }
    }
}

template <typename T, typename OutVec>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]);

template <>
__device__ __forceinline__ void store8<float, uint4>(float* p, const float (&v)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16, uint4>(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        ow[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = o;
}
template <>
__device__ __forceinline__ void store8<__half, uint4>(__half* p, const float (&v)[8]) {
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        ow[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = o;
}

// Fast path: 8 outputs per thread; needs out 16-byte aligned and packed 4-byte aligned.
template <typename T>
__global__ void __launch_bounds__(QTHREADS) dequantize_kernel(const uint32_t* __restrict__ packed32,
                                                              const float* __restrict__ absmax,
                                                              const float* __restrict__ code16, int64_t ngroups8,
                                                              int log2_groups_per_block, T* __restrict__ out) {
    __shared__ float s_code[16];
    if (threadIdx.x < 16) s_code[threadIdx.x] = code16[threadIdx.x];
    __syncthreads();
    for (int64_t t = (int64_t)blockIdx.x * QTHREADS + threadIdx.x; t < ngroups8; t += (int64_t)gridDim.x * QTHREADS) {
        const uint32_t word = ld_nc_u32(packed32 + t);
        const float am = __ldg(absmax + (t >> log2_groups_per_block));
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int shift = (i >> 1) * 8 + ((i & 1) ? 0 : 4);
            v[i] = __fmul_rn(s_code[(word >> shift) & 15u], am);
        }
        store8<T, uint4>(out + t * 8, v);
    }
}

template <typename T>
__global__ void dequantize_tail_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ absmax,
                                       const float* __restrict__ code16, int64_t first, int64_t numel, int blocksize,
                                       T* __restrict__ out) {
    for (int64_t i = first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < numel;
         i += (int64_t)gridDim.x * blockDim.x) {
        const uint8_t byte = packed[i >> 1];
        const int idx = (i & 1) ? (byte & 15) : (byte >> 4);
        out[i] = Elem<T>::from_f32(__fmul_rn(code16[idx], absmax[i / blocksize]));
    }
}

static int ilog2(int v) {
    int l = 0;
    while ((1 << l) < v) ++l;
    return l;
}

template <typename T>
static int quantize_typed(const T* w, int64_t numel, int blocksize, const float* code16, uint8_t* packed,
                          float* absmax, cudaStream_t stream) {
    const bool aligned = (reinterpret_cast<uintptr_t>(w) % 16 == 0) && (reinterpret_cast<uintptr_t>(packed) % 4 == 0);
    int64_t full_blocks = aligned ? numel / blocksize : 0;
    if (full_blocks > 0) {
        const int64_t ngroups8 = full_blocks * (blocksize / 8);
        int64_t want = (ngroups8 + QTHREADS - 1) / QTHREADS;
        const int64_t cap = (int64_t)sm_count() * 8;     // 8 resident CTAs per SM; the per-CTA threshold set-up is amortised over a long loop
        const int grid = (int)(want < cap ? want : cap);
        uint32_t* p32 = reinterpret_cast<uint32_t*>(packed);
#define NF4_Q_LAUNCH(G) quantize_kernel<T, G><<<grid, QTHREADS, 0, stream>>>(w, ngroups8, code16, p32, absmax)
        switch (blocksize) {
            case 64: NF4_Q_LAUNCH(8); break;
            case 128: NF4_Q_LAUNCH(16); break;
            case 256: NF4_Q_LAUNCH(32); break;
            case 512: NF4_Q_LAUNCH(64); break;
            case 1024: NF4_Q_LAUNCH(128); break;
            case 2048: NF4_Q_LAUNCH(256); break;
            default: full_blocks = 0; break;   // 4096: one thread block cannot hold a group; use the tail kernel
        }
#undef NF4_Q_LAUNCH
        NF4_CUDA_TRY(cudaGetLastError());
    }
    const int64_t nblocks = (numel + blocksize - 1) / blocksize;
    if (full_blocks < nblocks) {
        const int64_t rest = nblocks - full_blocks;
        const int threads = 128;
        int64_t want = (rest + threads - 1) / threads;
        const int64_t cap = (int64_t)sm_count() * 16;
        const int grid = (int)(want < cap ? want : cap);
        quantize_tail_kernel<T><<<grid, threads, 0, stream>>>(w, full_blocks, numel, blocksize, code16, packed, absmax);
        NF4_CUDA_TRY(cudaGetLastError());
    }
    return NF4_OK;
}

template <typename T>
static int dequantize_typed(const uint8_t* packed, const float* absmax, const float* code16, int64_t numel,
                            int blocksize, T* out, cudaStream_t stream) {
    const bool aligned = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && (reinterpret_cast<uintptr_t>(packed) % 4 == 0);
    const int64_t ngroups8 = aligned ? numel / 8 : 0;
    if (ngroups8 > 0) {
        int64_t want = (ngroups8 + QTHREADS - 1) / QTHREADS;
        const int64_t cap = (int64_t)sm_count() * 8 * 4;
        const int grid = (int)(want < cap ? want : cap);
        dequantize_kernel<T><<<grid, QTHREADS, 0, stream>>>(reinterpret_cast<const uint32_t*>(packed), absmax, code16,
                                                            ngroups8, ilog2(blocksize / 8), out);
        NF4_CUDA_TRY(cudaGetLastError());
    }
    if (ngroups8 * 8 < numel) {
        const int64_t rest = numel - ngroups8 * 8;
        const int threads = 128;
        int64_t want = (rest + threads - 1) / threads;
        const int64_t cap = (int64_t)sm_count() * 16;
        const int grid = (int)(want < cap ? want : cap);
        dequantize_tail_kernel<T><<<grid, threads, 0, stream>>>(packed, absmax, code16, ngroups8 * 8, numel, blocksize, out);
        NF4_CUDA_TRY(cudaGetLastError());
    }
    return NF4_OK;
}

static bool valid_blocksize(int b) { return b >= 64 && b <= 4096 && (b & (b - 1)) == 0; }

}  // namespace nf4

using namespace nf4;

extern "C" int nf4_b200_quantize(const void* w, int64_t numel, int w_dtype, int blocksize, const float* code16,
                                 uint8_t* packed, float* absmax, void* stream) {
    NF4_REQUIRE(numel >= 0, NF4_ERR_ARG, "quantize: numel %lld < 0", (long long)numel);
    NF4_REQUIRE(valid_blocksize(blocksize), NF4_ERR_ARG, "quantize: blocksize %d is not a power of two in [64, 4096]", blocksize);
    if (numel == 0) return NF4_OK;
    NF4_REQUIRE(w && code16 && packed && absmax, NF4_ERR_ARG, "quantize: null pointer");
    if (int rc = check_device()) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (w_dtype) {
        case NF4_F32: return quantize_typed(static_cast<const float*>(w), numel, blocksize, code16, packed, absmax, s);
        case NF4_F16: return quantize_typed(static_cast<const __half*>(w), numel, blocksize, code16, packed, absmax, s);
        case NF4_BF16: return quantize_typed(static_cast<const __nv_bfloat16*>(w), numel, blocksize, code16, packed, absmax, s);
    }
    set_error("quantize: unknown dtype code %d", w_dtype);
    return NF4_ERR_ARG;
}

extern "C" int nf4_b200_dequantize(const uint8_t* packed, const float* absmax, const float* code16, int64_t numel,
                                   int blocksize, void* out, int out_dtype, void* stream) {
    NF4_REQUIRE(numel >= 0, NF4_ERR_ARG, "dequantize: numel %lld < 0", (long long)numel);
    NF4_REQUIRE(valid_blocksize(blocksize), NF4_ERR_ARG, "dequantize: blocksize %d is not a power of two in [64, 4096]", blocksize);
    if (numel == 0) return NF4_OK;
    NF4_REQUIRE(packed && code16 && out && absmax, NF4_ERR_ARG, "dequantize: null pointer");
    if (int rc = check_device()) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (out_dtype) {
        case NF4_F32: return dequantize_typed(packed, absmax, code16, numel, blocksize, static_cast<float*>(out), s);
        case NF4_F16: return dequantize_typed(packed, absmax, code16, numel, blocksize, static_cast<__half*>(out), s);
        case NF4_BF16: return dequantize_typed(packed, absmax, code16, numel, blocksize, static_cast<__nv_bfloat16*>(out), s);
    }
    set_error("dequantize: unknown dtype code %d", out_dtype);
    return NF4_ERR_ARG;
}
