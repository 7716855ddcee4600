// Host-side plumbing of the C ABI: error strings, device checks, the linear dispatcher.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "nf4_common.cuh"

namespace nf4 {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("%s failed: %s", what, cudaGetErrorString(e));
    return NF4_ERR_CUDA;
}

struct DevInfo { int known; int major; int sms; };
static DevInfo g_dev[64];

static int dev_info(DevInfo** out) {
    int dev = 0;
    NF4_CUDA_TRY(cudaGetDevice(&dev));
    NF4_REQUIRE(dev >= 0 && dev < 64, NF4_ERR_LIMIT, "device ordinal %d above 63", dev);
    DevInfo& d = g_dev[dev];
    if (!d.known) {
        int major = 0, sms = 0;
        NF4_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        NF4_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        d.major = major;
        d.sms = sms;
        d.known = 1;
    }
    *out = &d;
    return NF4_OK;
}

int check_device() {
    DevInfo* d = nullptr;
    if (int rc = dev_info(&d)) return rc;
    NF4_REQUIRE(d->major == 10, NF4_ERR_ARCH, "this library is built for sm_100a only; current device is compute capability %d.x", d->major);
    return NF4_OK;
}

int sm_count() {
    DevInfo* d = nullptr;
    if (dev_info(&d)) return 148;
    return d->sms > 0 ? d->sms : 148;
}

bool gemv_supported(int64_t M, int64_t K, int64_t N, int blocksize, int dtype, const void* x, const void* packed,
                    const void* absmax);
bool gemm_supported(int64_t M, int64_t K, int64_t N, int blocksize, int dtype, const void* x, const void* packed,
                    const void* absmax, const void* y);
int gemm_min_m();

}  // namespace nf4

using namespace nf4;

static thread_local int g_last_path = 0;

extern "C" int nf4_b200_version(void) { return 100; }

extern "C" int nf4_b200_last_linear_path(void) { return g_last_path; }

extern "C" int nf4_b200_last_error(char* buf, int buflen) {
    const int n = (int)strlen(g_error);
    if (buf && buflen > 0) {
        const int c = n < buflen - 1 ? n : buflen - 1;
        memcpy(buf, g_error, (size_t)c);
        buf[c] = 0;
    }
    return n;
}

extern "C" int64_t nf4_b200_linear_workspace_bytes(int64_t M, int64_t N, int64_t K, int dtype) {
    if (dtype != NF4_BF16 || M < nf4::gemm_min_m() || K % 64 != 0) return 0;
    return nf4_b200_gemm_workspace_bytes(M, N, K);
}

extern "C" int nf4_b200_linear(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                               const float* code16, int64_t N, int blocksize, const void* bias, void* y, int dtype,
                               void* workspace, int64_t workspace_bytes, void* stream) {
    NF4_REQUIRE(M >= 0 && N >= 0 && K >= 0, NF4_ERR_ARG, "linear: negative extent M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
    NF4_REQUIRE(dtype == NF4_F32 || dtype == NF4_F16 || dtype == NF4_BF16, NF4_ERR_ARG, "linear: unknown dtype code %d", dtype);
    if (M == 0 || N == 0) return NF4_OK;
    NF4_REQUIRE(x && packed && absmax && code16 && y, NF4_ERR_ARG, "linear: null pointer");
    const bool gemm_ok = gemm_supported(M, K, N, blocksize, dtype, x, packed, absmax, y);
    if (!gemm_ok && gemv_supported(M, K, N, blocksize, dtype, x, packed, absmax)) {
        g_last_path = NF4_PATH_GEMV;
        return nf4_b200_gemv(x, M, K, packed, absmax, code16, N, bias, y, dtype, stream);
    }
    if (gemm_ok) {
        g_last_path = NF4_PATH_GEMM;
        return nf4_b200_gemm(x, M, K, packed, absmax, code16, N, bias, y, dtype, workspace, workspace_bytes, stream);
    }
    // fp16 with more than 16 rows: the tensor-core kernel is bf16 only; nf4_b200_gemm runs the fused GEMV once per
    // slab of 16 activation rows instead (the weight streams once per slab, still far ahead of the generic kernel)
    if (dtype == NF4_F16 && M > 16 && gemv_supported(16, K, N, blocksize, dtype, x, packed, absmax)) {
        g_last_path = NF4_PATH_GEMV_SLABS;
        return nf4_b200_gemm(x, M, K, packed, absmax, code16, N, bias, y, dtype, workspace, workspace_bytes, stream);
    }
    g_last_path = NF4_PATH_GENERIC;
    return nf4_b200_linear_generic(x, M, K, packed, absmax, code16, N, blocksize, bias, y, dtype, stream);
}
