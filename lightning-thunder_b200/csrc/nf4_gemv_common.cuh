// Pieces shared by the two fused dequant-GEMV kernels: the mma.sync wrapper and the
// conflict-free byte -> (16-bit, 16-bit) lookup table in shared memory.
#pragma once

#include "nf4_common.cuh"

namespace nf4 {

constexpr int GEMV_SMEM = 232448;          // 227 KB: the opt-in maximum per CTA
constexpr int LUT_WINDOW = 65536;          // 256 entries x 256 B, 64 KB aligned in the shared window

template <typename T> struct Mma;
template <> struct Mma<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                               const float (&c)[4]) {
        asm(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
    }
    // D = A*B with a zero accumulator (one register holds the zero)
    static __device__ __forceinline__ void run0(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
    }
    // D += A*B in place
    static __device__ __forceinline__ void acc(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};
template <> struct Mma<__half> {
    static __device__ __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                               const float (&c)[4]) {
        asm(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
    }
    static __device__ __forceinline__ void run0(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
    }
    static __device__ __forceinline__ void acc(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};

// one table lookup: byte `SEL` of w -> two 16-bit values
template <int SEL>
__device__ __forceinline__ uint32_t lut_lookup(uint32_t w, uint32_t window_lane) {
    const uint32_t addr = __byte_perm(w, window_lane, 0x7604 | (SEL << 4));
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}


// Fills the table: entry e (a packed byte) -> levels of its high and low nibble, one copy per lane.
// Called by `nwarps` warps (warp index `warp`); lut_ptr is the generic address of the window.
// `level` is code16[lane & 15], loaded by the caller as early as it can (one global latency, not 32).
template <typename T, int NWARPS>
__device__ __forceinline__ void lut_build(uint8_t* lut_ptr, float level, int warp, int lane) {
#pragma unroll
    for (int i = 0; i < 256 / NWARPS; ++i) {      // independent iterations: the shuffles and stores pipeline
        const int e = warp + i * NWARPS;
        const uint32_t v = Mma<T>::pack(__shfl_sync(0xffffffffu, level, e >> 4), __shfl_sync(0xffffffffu, level, e & 15));
        *reinterpret_cast<uint32_t*>(lut_ptr + e * 256 + lane * 4) = v;
    }
}

struct GemvOptions {
    int prologue = 0;             // 0 none, 1 rmsnorm(x) * norm_w, 2 silu(x[:, :K]) * x[:, K:]
    const void* norm_w = nullptr;
    float eps = 0.0f;
    int epilogue = 0;             // 0 none, 1 SwiGLU over (gate, up) row pairs (output has N/2 columns)
    bool pdl = false;             // launch with programmatic stream serialization
    bool dry_run = false;         // plan only: report whether the shape (and prologue) fits
    // weight the NEXT launch on this stream will read: each CTA pulls the head of its share into L2
    // once its own loads have been issued (fills the HBM idle time around the kernel boundary)
    // double-quantized absmax: uint8 indices [N*K/64], one fp32 scale per 256 of them, a device scalar offset
    // and the 256-entry table; the `absmax` argument of the call is then unused
    const uint8_t* dq_absmax_u8 = nullptr;
    const float* dq_scale2 = nullptr;
    const float* dq_offset = nullptr;
    const float* dq_code256 = nullptr;
    const uint8_t* next_packed = nullptr;
    const float* next_absmax = nullptr;
    int next_N = 0, next_K = 0;
};

// Staged (TMA ring) GEMV: launches and returns NF4_OK (or an error code); returns -1 if the shape does
// not fit the kernel, -2 if only the requested prologue does not fit.
template <typename T>
int gemv_staged_try(const void* x, int M, int K, const uint8_t* packed, const float* absmax, const float* code16, int N,
                    const void* bias, const void* residual, void* y, cudaStream_t stream, const GemvOptions& opt);

}  // namespace nf4
