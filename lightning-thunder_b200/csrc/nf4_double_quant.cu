// Double quantization of absmax (8-bit, blocks of 256, one fp32 scale per block and one global
// offset).  Not part of the reference (thunder/transforms/quantization.py:84 leaves it as a TODO);
// semantics are those of this library's CPU oracle:
//   offset = fp32( sum_fp64(absmax) / count );  r = absmax - offset;  scale2[b] = max |r| over block b;
//   u8 = index of the nearest entry of the sorted 256-entry table to r / scale2 (lower index wins a
//   tie; an all-zero block maps to the entry 0.0);  absmax' = fma(code256[u8], scale2, offset).
// The fp64 sum is exact (hence order-independent) whenever the values span fewer than 2^6 in
// magnitude for up to 2^23 blocks, which holds for absmax of real weights; outside that range the
// offset may differ from a sequential sum in its last bit.
#include "nf4_common.cuh"

namespace nf4 {

// one CTA, fixed summation order: thread-strided partial sums, then a shared-memory tree
__global__ void __launch_bounds__(1024) dq_offset_kernel(const float* __restrict__ absmax, int64_t n, float* __restrict__ offset) {
    __shared__ double s[1024];
    double acc = 0.0;
    for (int64_t i = threadIdx.x; i < n; i += 1024) acc += (double)absmax[i];
    s[threadIdx.x] = acc;
    __syncthreads();
    for (int w = 512; w > 0; w >>= 1) {
        if (threadIdx.x < w) s[threadIdx.x] += s[threadIdx.x + w];
        __syncthreads();
    }
    if (threadIdx.x == 0) *offset = n > 0 ? (float)(s[0] / (double)n) : 0.0f;
}

// one warp per block of 256 absmax values
__global__ void __launch_bounds__(256) dq_quantize_kernel(const float* __restrict__ absmax, int64_t n,
                                                          const float* __restrict__ code256,
                                                          const float* __restrict__ offset_p, uint8_t* __restrict__ out,
                                                          float* __restrict__ scale2) {
    __shared__ float s_thr[256];   // thr[i], i < 255: smallest v that maps to index i+1 rather than i
    __shared__ int s_zero;
    {
        const int i = threadIdx.x;
        if (i < 255) s_thr[i] = level_threshold(code256[i], code256[i + 1]);
        else s_thr[255] = __int_as_float(0x7f800000);
        if (i == 0) {
            int z = 0;
            for (int k = 0; k < 256; ++k) if (code256[k] == 0.0f) { z = k; break; }
            s_zero = z;
        }
    }
    __syncthreads();
    const float offset = *offset_p;
    const int lane = threadIdx.x & 31;
    const int64_t nb2 = (n + 255) / 256;
    for (int64_t b = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); b < nb2; b += (int64_t)gridDim.x * 8) {
        const int64_t base = b * 256 + lane * 8;
        float r[8];
        float am = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int64_t i = base + j;
            r[j] = i < n ? __fsub_rn(absmax[i], offset) : 0.0f;
            am = fmaxf(am, fabsf(r[j]));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        if (lane == 0) scale2[b] = am;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int64_t i = base + j;
            if (i < n) {
                uint32_t idx = (uint32_t)s_zero;
                if (am != 0.0f) {
                    const float v = __fdiv_rn(r[j], am);
                    idx = 0;                               // count of thresholds <= v, 8-step binary search
#pragma unroll
                    for (int step = 128; step > 0; step >>= 1)
                        if (v >= s_thr[idx + step - 1]) idx += step;
                }
                out[i] = (uint8_t)idx;
            }
        }
    }
}

__global__ void dq_dequantize_kernel(const uint8_t* __restrict__ u8, const float* __restrict__ scale2,
                                     const float* __restrict__ offset_p, const float* __restrict__ code256, int64_t n,
                                     float* __restrict__ absmax) {
    __shared__ float s_code[256];
    if (threadIdx.x < 256) s_code[threadIdx.x] = code256[threadIdx.x];
    __syncthreads();
    const float offset = *offset_p;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        absmax[i] = __fmaf_rn(s_code[u8[i]], scale2[i >> 8], offset);
}

}  // namespace nf4

using namespace nf4;

extern "C" int nf4_b200_dq_quantize(const float* absmax, int64_t nblocks, const float* code256, uint8_t* absmax_u8,
                                    float* scale2, float* offset, void* stream) {
    NF4_REQUIRE(nblocks >= 0, NF4_ERR_ARG, "dq_quantize: nblocks %lld < 0", (long long)nblocks);
    NF4_REQUIRE(code256 && offset, NF4_ERR_ARG, "dq_quantize: null pointer");
    if (int rc = check_device()) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    dq_offset_kernel<<<1, 1024, 0, s>>>(absmax, nblocks, offset);
    NF4_CUDA_TRY(cudaGetLastError());
    if (nblocks == 0) return NF4_OK;
    NF4_REQUIRE(absmax && absmax_u8 && scale2, NF4_ERR_ARG, "dq_quantize: null pointer");
    const int64_t nb2 = (nblocks + 255) / 256;
    int64_t want = (nb2 + 7) / 8;
    const int64_t cap = (int64_t)sm_count() * 8;
    dq_quantize_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, s>>>(absmax, nblocks, code256, offset, absmax_u8, scale2);
    NF4_CUDA_TRY(cudaGetLastError());
    return NF4_OK;
}

extern "C" int nf4_b200_dq_dequantize(const uint8_t* absmax_u8, const float* scale2, const float* offset,
                                      const float* code256, int64_t nblocks, float* absmax, void* stream) {
    NF4_REQUIRE(nblocks >= 0, NF4_ERR_ARG, "dq_dequantize: nblocks %lld < 0", (long long)nblocks);
    if (nblocks == 0) return NF4_OK;
    NF4_REQUIRE(absmax_u8 && scale2 && offset && code256 && absmax, NF4_ERR_ARG, "dq_dequantize: null pointer");
    if (int rc = check_device()) return rc;
    int64_t want = (nblocks + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    dq_dequantize_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        absmax_u8, scale2, offset, code256, nblocks, absmax);
    NF4_CUDA_TRY(cudaGetLastError());
    return NF4_OK;
}

namespace nf4 {
int gemv_dq_try(const void* x, int64_t M, int64_t K, const uint8_t* packed, const uint8_t* absmax_u8, const float* scale2,
                const float* offset, const float* code256, const float* code16, int64_t N, const void* bias, void* y,
                int dtype, cudaStream_t stream);
}

extern "C" int64_t nf4_b200_linear_dq_workspace_bytes(int64_t N, int64_t K) { return ((N * K + 63) / 64) * 4; }

extern "C" int nf4_b200_linear_dq(const void* x, int64_t M, int64_t K, const uint8_t* packed, const uint8_t* absmax_u8,
                                  const float* scale2, const float* offset, const float* code256, const float* code16,
                                  int64_t N, const void* bias, void* y, int dtype, void* workspace, int64_t workspace_bytes,
                                  void* stream) {
    NF4_REQUIRE(M >= 0 && N >= 0 && K >= 0, NF4_ERR_ARG, "linear_dq: negative extent");
    if (M == 0 || N == 0) return NF4_OK;
    NF4_REQUIRE(x && packed && absmax_u8 && scale2 && offset && code256 && code16 && y, NF4_ERR_ARG, "linear_dq: null pointer");
    // up to 16 activation rows: the fused GEMV expands the 8-bit absmax inside its stages (no workspace traffic)
    if (int rc = check_device()) return rc;
    {
        const int rc = gemv_dq_try(x, M, K, packed, absmax_u8, scale2, offset, code256, code16, N, bias, y, dtype,
                                   static_cast<cudaStream_t>(stream));
        if (rc >= 0) return rc;
    }
    const int64_t nblocks = (N * K + 63) / 64;
    NF4_REQUIRE(workspace && workspace_bytes >= nblocks * 4, NF4_ERR_WORKSPACE,
                "linear_dq: workspace of %lld bytes, need %lld (nf4_b200_linear_dq_workspace_bytes)",
                (long long)workspace_bytes, (long long)(nblocks * 4));
    float* am = static_cast<float*>(workspace);
    if (int rc = nf4_b200_dq_dequantize(absmax_u8, scale2, offset, code256, nblocks, am, stream)) return rc;
    return nf4_b200_linear(x, M, K, packed, am, code16, N, 64, bias, y, dtype, nullptr, 0, stream);
}
