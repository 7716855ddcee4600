// Prefill-regime dequant-GEMM (M > 16).
#include "nf4_common.cuh"

namespace nf4 {

bool gemv_supported(int64_t M, int64_t K, int64_t N, int blocksize, int dtype, const void* x, const void* packed,
                    const void* absmax);

bool gemm_supported(int64_t M, int64_t K, int64_t N, int blocksize, int dtype, const void* x, const void* packed,
                    const void* absmax, const void* y) {
    (void)y;
    return M > 16 && gemv_supported(16, K, N, blocksize, dtype, x, packed, absmax);
}

}  // namespace nf4

using namespace nf4;

extern "C" int nf4_b200_gemm(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                             const float* code16, int64_t N, const void* bias, void* y, int dtype, void* workspace,
                             int64_t workspace_bytes, void* stream) {
    (void)workspace; (void)workspace_bytes;
    NF4_REQUIRE(x && packed && absmax && code16 && y, NF4_ERR_ARG, "gemm: null pointer");
    NF4_REQUIRE(M >= 1, NF4_ERR_ARG, "gemm: M=%lld < 1", (long long)M);
    NF4_REQUIRE(gemm_supported(M > 16 ? M : 17, K, N, 64, dtype, x, packed, absmax, y), NF4_ERR_ARG,
                "gemm: needs K %% 64 == 0, fp16/bf16, 16-byte aligned x");
    const int64_t esz = 2;
    for (int64_t m0 = 0; m0 < M; m0 += 16) {
        const int64_t mc = (M - m0) < 16 ? (M - m0) : 16;
        int rc = nf4_b200_gemv(static_cast<const uint8_t*>(x) + m0 * K * esz, mc, K, packed, absmax, code16, N, bias,
                               static_cast<uint8_t*>(y) + m0 * N * esz, dtype, stream);
        if (rc) return rc;
    }
    return NF4_OK;
}
