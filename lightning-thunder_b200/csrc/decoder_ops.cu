// The small kernels that sit between the NF4 linears in a Llama-shaped decode step (bf16
// activations, fp32 arithmetic): RMSNorm, rotary embedding + KV-cache append, single-query
// grouped attention over the cache, SiLU(gate)*up, embedding lookup and greedy argmax.  They exist
// so that a decode step is a short chain of launches that can be captured in one CUDA graph; the
// reference leaves this glue to its trace executors (nvFuser / torch eager), which are not part
// of this path.
#include <cfloat>

#include "nf4_common.cuh"

namespace nf4 {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- RMSNorm: y[r][:] = x[r][:] * rsqrt(mean(x^2) + eps) * w[:] ---------------------------------
__global__ void __launch_bounds__(256) rmsnorm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                      bf16* __restrict__ y, int D, float eps) {
    __shared__ float s_part[8];
    const bf16* xr = x + (int64_t)blockIdx.x * D;
    bf16* yr = y + (int64_t)blockIdx.x * D;
    float ss = 0.0f;
    for (int i = threadIdx.x * 2; i < D; i += 512) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + i));
        ss += v.x * v.x + v.y * v.y;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += s_part[i];
    const float r = rsqrtf(tot / (float)D + eps);
    for (int i = threadIdx.x * 2; i < D; i += 512) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + i));
        const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + i));
        *reinterpret_cast<__nv_bfloat162*>(yr + i) = __floats2bfloat162_rn(v.x * r * g.x, v.y * r * g.y);
    }
}

// Status word of the kernels that index the KV cache with a position read from device memory:
// [0] first error code (9 = a position outside [0, S_max)), [1] batch row, [2] the position, [3] count.
// Such a row writes nothing to the cache and attends to nothing (its output is zero).
__device__ unsigned int g_attn_error[4];

__device__ __forceinline__ bool position_in_range(int pos, int S_max) { return (unsigned)pos < (unsigned)S_max; }

__device__ __noinline__ void report_bad_position(int b, int pos) {
    if (atomicCAS(&g_attn_error[0], 0u, 9u) == 0u) {
        g_attn_error[1] = (unsigned)b;
        g_attn_error[2] = (unsigned)pos;
    }
    atomicAdd(&g_attn_error[3], 1u);
}

__device__ __forceinline__ bool position_ok(int pos, int S_max, int b) {
    const bool ok = position_in_range(pos, S_max);
    if (!ok && threadIdx.x == 0) report_bad_position(b, pos);
    return ok;
}

// ---- rotary embedding on q and k (interleaved pairs) + append k, v to the cache ---------------
// qkv [B][(Hq + 2*Hkv) * Dh] as produced by the fused QKV linear; q_out [B][Hq*Dh];
// k_cache / v_cache [B][Hkv][S_max][Dh]; positions[B] = index of the token being written.
__global__ void rope_append_kernel(const bf16* __restrict__ qkv, const int* __restrict__ positions,
                                   bf16* __restrict__ q_out, bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                                   int Hq, int Hkv, int Dh, int S_max, float theta) {
    const int b = blockIdx.y;
    const int head = blockIdx.x;              // 0..Hq+2*Hkv-1
    const int pos = positions[b];
    const bool pos_ok = position_ok(pos, S_max, b);
    const bf16* src = qkv + ((int64_t)b * (Hq + 2 * Hkv) + head) * Dh;
    const int i = threadIdx.x;                // pair index, Dh/2 threads
    if (i >= Dh / 2) return;
    if (!pos_ok && head >= Hq) return;        // nothing is written outside the cache
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + 2 * i));
    if (head < Hq + Hkv) {
        const float inv_freq = powf(theta, -2.0f * (float)i / (float)Dh);
        float sn, cs;
        sincosf((float)pos * inv_freq, &sn, &cs);
        const __nv_bfloat162 r = __floats2bfloat162_rn(v.x * cs - v.y * sn, v.x * sn + v.y * cs);
        if (head < Hq) {
            *reinterpret_cast<__nv_bfloat162*>(q_out + ((int64_t)b * Hq + head) * Dh + 2 * i) = r;
        } else {
            const int h = head - Hq;
            *reinterpret_cast<__nv_bfloat162*>(k_cache + (((int64_t)b * Hkv + h) * S_max + pos) * Dh + 2 * i) = r;
        }
    } else {
        const int h = head - Hq - Hkv;
        *reinterpret_cast<__nv_bfloat162*>(v_cache + (((int64_t)b * Hkv + h) * S_max + pos) * Dh + 2 * i) =
            __floats2bfloat162_rn(v.x, v.y);
    }
}

// ---- the same for a whole prompt: qkv [B][T][(Hq + 2*Hkv) * Dh], positions[T] (shared by the sequences) -------
// q goes out in attention layout q_out [B][Hq][T][Dh]; rotated k and v go to cache rows positions[t].  One CTA per
// (token, sequence); 256 is a multiple of Dh/2, so a thread keeps one pair index and computes its angle once.
__global__ void __launch_bounds__(256) rope_prefill_kernel(const bf16* __restrict__ qkv, const int* __restrict__ positions,
                                                           bf16* __restrict__ q_out, bf16* __restrict__ k_cache,
                                                           bf16* __restrict__ v_cache, int T, int Hq, int Hkv, int Dh,
                                                           int S_max, float theta) {
    const int t = blockIdx.x, b = blockIdx.y;
    const int pos = positions[t];
    const bool pos_ok = position_in_range(pos, S_max);
    const int half = Dh >> 1;
    const int i = threadIdx.x % half;
    const float inv_freq = powf(theta, -2.0f * (float)i / (float)Dh);
    float sn, cs;
    sincosf((float)pos * inv_freq, &sn, &cs);
    const int H = Hq + 2 * Hkv;
    const bf16* src = qkv + ((int64_t)b * T + t) * H * Dh;
    for (int e = threadIdx.x; e < H * half; e += 256) {
        const int head = e / half;
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + head * Dh + 2 * i));
        if (head < Hq) {
            *reinterpret_cast<__nv_bfloat162*>(q_out + (((int64_t)b * Hq + head) * T + t) * Dh + 2 * i) =
                __floats2bfloat162_rn(v.x * cs - v.y * sn, v.x * sn + v.y * cs);
        } else if (pos_ok) {
            if (head < Hq + Hkv) {
                *reinterpret_cast<__nv_bfloat162*>(k_cache + (((int64_t)b * Hkv + head - Hq) * S_max + pos) * Dh + 2 * i) =
                    __floats2bfloat162_rn(v.x * cs - v.y * sn, v.x * sn + v.y * cs);
            } else {
                *reinterpret_cast<__nv_bfloat162*>(v_cache + (((int64_t)b * Hkv + head - Hq - Hkv) * S_max + pos) * Dh + 2 * i) =
                    __floats2bfloat162_rn(v.x, v.y);
            }
        }
    }
    if (!pos_ok && threadIdx.x == 0) report_bad_position(b, pos);
}

// Merge of the per-split partial results of one (batch row, query head): `base` points at
// [nsplit][Dh + 2] floats (Dh unnormalised outputs, max, sum).  One warp per head; lane s fetches
// the (max, sum) of split s, the weights are shared by shuffle and every lane owns 4 output dims,
// whose nsplit partial vectors are fetched together.  nsplit <= 32.
__device__ __forceinline__ void merge_splits_warp(const float* __restrict__ base, int nsplit, int lane, bf16* __restrict__ dst) {
    constexpr int Dh = 128;
    float mi = -FLT_MAX, li = 0.0f;
    if (lane < nsplit) {
        mi = __ldcg(base + lane * (Dh + 2) + Dh);
        li = __ldcg(base + lane * (Dh + 2) + Dh + 1);
    }
    float mm = mi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
    const float ci = lane < nsplit ? __expf(mi - mm) : 0.0f;
    float ll = li * ci;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ll += __shfl_xor_sync(0xffffffffu, ll, o);
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int s0 = 0; s0 < nsplit; s0 += 8) {
        float2 lo[8], hi[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int s = s0 + u;
            lo[u] = make_float2(0.0f, 0.0f);
            hi[u] = make_float2(0.0f, 0.0f);
            if (s < nsplit) {   // rows are (Dh+2) floats apart: 8-byte aligned, not 16
                lo[u] = __ldcg(reinterpret_cast<const float2*>(base + s * (Dh + 2) + lane * 4));
                hi[u] = __ldcg(reinterpret_cast<const float2*>(base + s * (Dh + 2) + lane * 4 + 2));
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float c = __shfl_sync(0xffffffffu, ci, (s0 + u) & 31);
            acc[0] += lo[u].x * c; acc[1] += lo[u].y * c; acc[2] += hi[u].x * c; acc[3] += hi[u].y * c;
        }
    }
    const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;
    *reinterpret_cast<__nv_bfloat162*>(dst + lane * 4) = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv);
    *reinterpret_cast<__nv_bfloat162*>(dst + lane * 4 + 2) = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
}

// ---- attention over a range of cached positions on the tensor cores ------------------------------
// One warp walks tiles of 16 positions: K and V rows are copied coalesced into the warp's shared-memory
// tile (16 rows x 256 B, 16-byte chunks XOR-swizzled with the row so ldmatrix is conflict-free), scores
// S = Q.K^T come from mma.sync m16n8k16 with the G <= 8 query heads of the group as rows 0..G-1 of the A
// operand (rows 8..15 stay zero), the online softmax runs on the accumulator fragments (a quad of lanes
// owns a head's 16 scores), and O += P.V takes P straight from those fragments and V through
// ldmatrix.trans.  Per position: 2 MMAs instead of 64 FMAs and 40 shuffles.
// Results of the warp: w_m[h], w_l[h], w_o[h][128] (unnormalised), in the warp's tile memory (w_o aliases
// the tiles, which are dead by then).
constexpr int AT_TILE = 16;                 // positions per tile
constexpr int AT_TILE_BYTES = AT_TILE * 256;
constexpr int AT_WARP_BYTES = 4 * AT_TILE_BYTES;     // per warp: two buffers of (K tile + V tile)
// dynamic shared memory of the attention kernels: 4 warps of tiles, the group's queries, the warps' max / sum, a flag
constexpr int AT_SMEM_BYTES = 4 * AT_WARP_BYTES + 8 * 128 * 2 + 2 * 4 * 8 * 4 + 16;

__device__ __forceinline__ void at_ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void at_ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void at_mma(float (&d)[2], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    // rows 8..15 of A (a1, a3) are zero, so rows 8..15 of the result are zero too and are not kept
    float x2, x3;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};"
                 : "+f"(d[0]), "+f"(d[1]), "=f"(x2), "=f"(x3) : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void at_cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
    // src_bytes = 0 fills the 16 bytes with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ uint32_t at_pack(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// q_s: bf16 [G][128] in shared memory (rotated, not scaled).  pos_new >= 0: that row of the cache is being
// written by this very kernel; its values come from knew/vnew (this lane's dims 4*lane..4*lane+3) instead.
template <int G>
__device__ __forceinline__ void attend_range(const bf16* __restrict__ kb, const bf16* __restrict__ vb, int s_begin, int s_end,
                                             int pos_new, const float (&knew)[4], const float (&vnew)[4],
                                             const bf16* q_s, float scale, uint8_t* tiles, float* w_m, float* w_l, float* w_o,
                                             int warp, int lane) {
    const int g = lane >> 2, q = lane & 3;
    const uint32_t k_u32 = (uint32_t)__cvta_generic_to_shared(tiles);
    // A fragments of Q for the 8 k-steps of 16 dims
    uint32_t qa0[8], qa2[8];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
        qa0[kk] = g < G ? *reinterpret_cast<const uint32_t*>(q_s + g * 128 + 16 * kk + 2 * q) : 0u;
        qa2[kk] = g < G ? *reinterpret_cast<const uint32_t*>(q_s + g * 128 + 16 * kk + 8 + 2 * q) : 0u;
    }
    float m = -FLT_MAX, l = 0.0f;
    float o[16][2];
#pragma unroll
    for (int t = 0; t < 16; ++t) { o[t][0] = 0.0f; o[t][1] = 0.0f; }

    // tiles are double-buffered: the asynchronous copy of the next tile runs under the MMAs of this one
    auto issue = [&](int s0, int buf) {
        const uint32_t kd = k_u32 + (uint32_t)(buf * 2 * AT_TILE_BYTES), vd = kd + AT_TILE_BYTES;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int idx = it * 32 + lane, r = idx >> 4, c = idx & 15, sp = s0 + r;
            const bool ok = sp < s_end && sp != pos_new;
            const int64_t off = ok ? (int64_t)sp * 128 + c * 8 : 0;
            const uint32_t dst = (uint32_t)(r * 256 + ((c ^ (r & 7)) << 4));
            at_cp_async16(kd + dst, kb + off, ok ? 16u : 0u);
            at_cp_async16(vd + dst, vb + off, ok ? 16u : 0u);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    int buf = 0;
    const int first = s_begin + warp * AT_TILE;
    if (first < s_end) issue(first, 0);
    for (int s0 = first; s0 < s_end; s0 += 4 * AT_TILE, buf ^= 1) {
        const int next = s0 + 4 * AT_TILE;
        if (next < s_end) {
            issue(next, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();
        uint8_t* const kt = tiles + buf * 2 * AT_TILE_BYTES;
        const uint32_t kt_u32 = k_u32 + (uint32_t)(buf * 2 * AT_TILE_BYTES), vt_u32 = kt_u32 + AT_TILE_BYTES;
        if (pos_new >= s0 && pos_new < s0 + AT_TILE && pos_new < s_end) {
            const int r = pos_new - s0;
            const int off = r * 256 + (((lane >> 1) ^ (r & 7)) << 4) + (lane & 1) * 8;
            *reinterpret_cast<uint2*>(kt + off) = make_uint2(at_pack(knew[0], knew[1]), at_pack(knew[2], knew[3]));
            *reinterpret_cast<uint2*>(kt + AT_TILE_BYTES + off) = make_uint2(at_pack(vnew[0], vnew[1]), at_pack(vnew[2], vnew[3]));
            __syncwarp();
        }
        // ---- S = Q.K^T: two n-tiles of 8 positions, 8 k-steps
        float sc[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            sc[j][0] = 0.0f; sc[j][1] = 0.0f;
#pragma unroll
            for (int kp = 0; kp < 4; ++kp) {
                const int r = 8 * j + (lane & 7), chunk = 4 * kp + (lane >> 3);
                uint32_t b[4];
                at_ldmatrix_x4(kt_u32 + (uint32_t)(r * 256 + ((chunk ^ (r & 7)) << 4)), b);
                at_mma(sc[j], qa0[2 * kp], qa2[2 * kp], b[0], b[1]);
                at_mma(sc[j], qa0[2 * kp + 1], qa2[2 * kp + 1], b[2], b[3]);
            }
        }
        // ---- online softmax on row g (this quad): columns 8j + 2q, 8j + 2q + 1
        float p[2][2];
        float tmax = -FLT_MAX;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int sp = s0 + 8 * j + 2 * q + e;
                p[j][e] = sp < s_end ? sc[j][e] * scale : -FLT_MAX;
                tmax = fmaxf(tmax, p[j][e]);
            }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        const float mn = fmaxf(m, tmax);
        const float corr = __expf(m - mn);
        float tsum = 0.0f;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                p[j][e] = p[j][e] > -FLT_MAX ? __expf(p[j][e] - mn) : 0.0f;
                tsum += p[j][e];
            }
        tsum += __shfl_xor_sync(0xffffffffu, tsum, 1);
        tsum += __shfl_xor_sync(0xffffffffu, tsum, 2);
        l = l * corr + tsum;
        m = mn;
        const uint32_t pa0 = at_pack(p[0][0], p[0][1]), pa2 = at_pack(p[1][0], p[1][1]);
        // ---- O = O * corr + P.V: 16 n-tiles of 8 dims, one k-step of 16 positions
#pragma unroll
        for (int tp = 0; tp < 8; ++tp) {
            const int mi = lane >> 3, r = (mi & 1) * 8 + (lane & 7), chunk = 2 * tp + (mi >> 1);
            uint32_t b[4];
            at_ldmatrix_x4_trans(vt_u32 + (uint32_t)(r * 256 + ((chunk ^ (r & 7)) << 4)), b);
            o[2 * tp][0] *= corr; o[2 * tp][1] *= corr;
            o[2 * tp + 1][0] *= corr; o[2 * tp + 1][1] *= corr;
            at_mma(o[2 * tp], pa0, pa2, b[0], b[1]);
            at_mma(o[2 * tp + 1], pa0, pa2, b[2], b[3]);
        }
        __syncwarp();       // the other buffer is refilled at the top of the next iteration
    }
    __syncwarp();
    if (g < G) {
#pragma unroll
        for (int t = 0; t < 16; ++t) {
            w_o[g * 128 + 8 * t + 2 * q] = o[t][0];
            w_o[g * 128 + 8 * t + 2 * q + 1] = o[t][1];
        }
        if (q == 0) { w_m[g] = m; w_l[g] = l; }
    }
}

// ---- single-query attention over the cache, split along the sequence --------------------------
// One CTA (4 warps) per (kv head, batch row, split); Dh = 128.  The G = Hq/Hkv query heads of the group
// share the K/V stream: each warp runs attend_range over every 4th tile of the split, the 4 warps'
// (max, sum, unnormalised output) are merged in shared memory, and the split's partial result goes
// to `ws` [B][Hq][nsplit][Dh + 2] fp32; attn_combine_kernel merges the splits.
template <int G>
__global__ void __launch_bounds__(128) attn_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache,
                                                          const bf16* __restrict__ v_cache,
                                                          const int* __restrict__ positions, float* __restrict__ ws,
                                                          int Hq, int Hkv, int S_max, int nsplit, float scale) {
    constexpr int Dh = 128;
    const int hk = blockIdx.x, b = blockIdx.y, sp = blockIdx.z;
    const int len = position_ok(positions[b], S_max, b) ? positions[b] + 1 : 0;    // attend to [0, pos]
    const int chunk = (len + nsplit - 1) / nsplit;
    const int s_begin = sp * chunk;
    const int s_end = min(len, s_begin + chunk);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // per warp: two buffers of K tile + V tile, reused for the warp's unnormalised output [G][128] fp32
    extern __shared__ __align__(128) uint8_t at_smem[];
    uint8_t (*s_tiles)[AT_WARP_BYTES] = reinterpret_cast<uint8_t (*)[AT_WARP_BYTES]>(at_smem);
    bf16* const s_q = reinterpret_cast<bf16*>(at_smem + 4 * AT_WARP_BYTES);
    float (*s_m)[8] = reinterpret_cast<float (*)[8]>(at_smem + 4 * AT_WARP_BYTES + 2048);
    float (*s_l)[8] = s_m + 4;
    for (int i = threadIdx.x; i < G * Dh / 2; i += 128)
        reinterpret_cast<uint32_t*>(s_q)[i] = reinterpret_cast<const uint32_t*>(q + ((int64_t)b * Hq + hk * G) * Dh)[i];
    __syncthreads();
    const bf16* kb = k_cache + ((int64_t)b * Hkv + hk) * S_max * Dh;
    const bf16* vb = v_cache + ((int64_t)b * Hkv + hk) * S_max * Dh;
    const float none[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    attend_range<G>(kb, vb, s_begin, s_end, -1, none, none, s_q, scale, s_tiles[warp], s_m[warp], s_l[warp],
                    reinterpret_cast<float*>(s_tiles[warp]), warp, lane);
    // merge the 4 warps
    auto s_o = [&](int w, int h, int d) -> float { return reinterpret_cast<const float*>(s_tiles[w])[h * Dh + d]; };
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * Dh; idx += 128) {
        const int h = idx / Dh, d = idx - h * Dh;
        float mm = -FLT_MAX;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, s_m[w][h]);
        float ll = 0.0f, oo = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float c = __expf(s_m[w][h] - mm);
            ll += s_l[w][h] * c;
            oo += s_o(w, h, d) * c;
        }
        float* dst = ws + (((int64_t)b * Hq + hk * G + h) * nsplit + sp) * (Dh + 2);
        dst[d] = oo;
        if (d == 0) { dst[Dh] = mm; dst[Dh + 1] = ll; }
    }
}

__global__ void __launch_bounds__(128) attn_combine_kernel(const float* __restrict__ ws, bf16* __restrict__ out,
                                                           int nsplit, int nheads_total) {
    constexpr int Dh = 128;
    const int bh = blockIdx.x * 4 + (threadIdx.x >> 5);       // b * Hq + head, one warp each
    if (bh >= nheads_total) return;
    merge_splits_warp(ws + (int64_t)bh * nsplit * (Dh + 2), nsplit, threadIdx.x & 31, out + (int64_t)bh * Dh);
}

// ---- rotary embedding + KV append + split attention + merge of the splits, one launch ----------
// Same arithmetic as rope_append_kernel + attn_decode_kernel + attn_combine_kernel (values are
// rounded to bf16 at the same points), one CTA per (kv head, batch row, split).  The split that
// owns the current position rotates the new key, writes key and value to the cache and uses them
// from registers; the last CTA of a (batch row, kv head) to finish -- found with a counter that the
// kernel leaves at zero again -- merges the partial results.
template <int G>
__global__ void __launch_bounds__(128) attn_fused_kernel(const bf16* __restrict__ qkv, const int* __restrict__ positions,
                                                         bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                                                         bf16* __restrict__ out, float* __restrict__ ws,
                                                         unsigned int* __restrict__ counters, int Hq, int Hkv, int S_max,
                                                         int nsplit, float scale, float theta) {
    constexpr int Dh = 128;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int hk = blockIdx.x, b = blockIdx.y, sp = blockIdx.z;
    const int pos = positions[b];
    const bool pos_ok = position_in_range(pos, S_max);    // reported beside the arrival counter, off the start-up path
    const int len = pos_ok ? pos + 1 : 0;
    const int chunk = (len + nsplit - 1) / nsplit;
    const int s_begin = sp * chunk;
    const int s_end = min(len, s_begin + chunk);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bf16* row = qkv + (int64_t)b * (Hq + 2 * Hkv) * Dh;

    // rotation of this lane's two pairs (dims 4*lane .. 4*lane+3)
    float cs[2], sn[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const float inv_freq = powf(theta, -2.0f * (float)(2 * lane + j) / (float)Dh);
        sincosf((float)pos * inv_freq, &sn[j], &cs[j]);
    }
    // positions and the rotation angles do not come from the predecessor grid (the QKV projection); qkv does
    asm volatile("griddepcontrol.wait;" ::: "memory");
    auto rotate = [&](const bf16* src, float (&r)[4]) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + lane * 4));
        const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + lane * 4 + 2));
        const float2 ra = __bfloat1622float2(__floats2bfloat162_rn(a.x * cs[0] - a.y * sn[0], a.x * sn[0] + a.y * cs[0]));
        const float2 rc = __bfloat1622float2(__floats2bfloat162_rn(c.x * cs[1] - c.y * sn[1], c.x * sn[1] + c.y * cs[1]));
        r[0] = ra.x; r[1] = ra.y; r[2] = rc.x; r[3] = rc.y;
    };
    // per warp: two buffers of K tile + V tile, reused for the warp's unnormalised output [G][128] fp32
    extern __shared__ __align__(128) uint8_t at_smem[];
    uint8_t (*s_tiles)[AT_WARP_BYTES] = reinterpret_cast<uint8_t (*)[AT_WARP_BYTES]>(at_smem);
    bf16* const s_q = reinterpret_cast<bf16*>(at_smem + 4 * AT_WARP_BYTES);
    float (*s_m)[8] = reinterpret_cast<float (*)[8]>(at_smem + 4 * AT_WARP_BYTES + 2048);
    float (*s_l)[8] = s_m + 4;
    int& s_last = *reinterpret_cast<int*>(at_smem + 4 * AT_WARP_BYTES + 2048 + 256);
    for (int h = warp; h < G; h += 4) {         // rotated queries of the group, as the A operand's source
        float r[4];
        rotate(row + (hk * G + h) * Dh, r);
        *reinterpret_cast<__nv_bfloat162*>(s_q + h * Dh + lane * 4) = __floats2bfloat162_rn(r[0], r[1]);
        *reinterpret_cast<__nv_bfloat162*>(s_q + h * Dh + lane * 4 + 2) = __floats2bfloat162_rn(r[2], r[3]);
    }
    __syncthreads();
    const bool owner = pos_ok && pos >= s_begin && pos < s_end;
    float knew[4] = {0, 0, 0, 0}, vnew[4] = {0, 0, 0, 0};
    bf16* kb = k_cache + ((int64_t)b * Hkv + hk) * S_max * Dh;
    bf16* vb = v_cache + ((int64_t)b * Hkv + hk) * S_max * Dh;
    if (owner) {
        rotate(row + (Hq + hk) * Dh, knew);
        const bf16* vsrc = row + (Hq + Hkv + hk) * Dh + lane * 4;
        const uint2 vr = *reinterpret_cast<const uint2*>(vsrc);
        const float2 v0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vr.x));
        const float2 v1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vr.y));
        vnew[0] = v0.x; vnew[1] = v0.y; vnew[2] = v1.x; vnew[3] = v1.y;
        if (warp == 0) {
            *reinterpret_cast<__nv_bfloat162*>(kb + (int64_t)pos * Dh + lane * 4) = __floats2bfloat162_rn(knew[0], knew[1]);
            *reinterpret_cast<__nv_bfloat162*>(kb + (int64_t)pos * Dh + lane * 4 + 2) = __floats2bfloat162_rn(knew[2], knew[3]);
            *reinterpret_cast<uint2*>(vb + (int64_t)pos * Dh + lane * 4) = vr;
        }
    }
    attend_range<G>(kb, vb, s_begin, s_end, owner ? pos : -1, knew, vnew, s_q, scale, s_tiles[warp], s_m[warp], s_l[warp],
                    reinterpret_cast<float*>(s_tiles[warp]), warp, lane);
    auto s_o = [&](int w, int h, int d) -> float { return reinterpret_cast<const float*>(s_tiles[w])[h * Dh + d]; };
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * Dh; idx += 128) {
        const int h = idx / Dh, d = idx - h * Dh;
        float mm = -FLT_MAX;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, s_m[w][h]);
        float ll = 0.0f, oo = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float c = __expf(s_m[w][h] - mm);
            ll += s_l[w][h] * c;
            oo += s_o(w, h, d) * c;
        }
        float* dst = ws + (((int64_t)b * Hq + hk * G + h) * nsplit + sp) * (Dh + 2);
        dst[d] = oo;
        if (d == 0) { dst[Dh] = mm; dst[Dh + 1] = ll; }
    }
    // ---- the last split to arrive merges ---------------------------------------------------------
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!pos_ok) report_bad_position(b, pos);
        const unsigned int old = atomicAdd(&counters[b * Hkv + hk], 1u);
        s_last = (old == (unsigned int)(nsplit - 1)) ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int h = warp; h < G; h += 4) {
        const int64_t bh = (int64_t)b * Hq + hk * G + h;
        merge_splits_warp(ws + bh * nsplit * (Dh + 2), nsplit, lane, out + bh * Dh);
    }
    if (threadIdx.x == 0) counters[b * Hkv + hk] = 0u;
}

// ---- h[r][i] = silu(gu[r][i]) * gu[r][F + i] -----------------------------------------------------
__global__ void silu_mul_kernel(const bf16* __restrict__ gu, bf16* __restrict__ h, int F, int64_t total_pairs, int interleaved) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;     // pair index over [rows][F/2]
    if (t >= total_pairs) return;
    const int64_t r = t / (F / 2);
    const int i = (int)(t - r * (F / 2)) * 2;
    float2 gte, up;
    if (interleaved) {   // (gate_i, up_i, gate_i+1, up_i+1) are adjacent
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gu + r * 2 * F + 2 * i));
        const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gu + r * 2 * F + 2 * i + 2));
        gte = make_float2(a.x, c.x);
        up = make_float2(a.y, c.y);
    } else {
        gte = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gu + r * 2 * F + i));
        up = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gu + r * 2 * F + F + i));
    }
    const float a = gte.x / (1.0f + __expf(-gte.x)) * up.x;
    const float c = gte.y / (1.0f + __expf(-gte.y)) * up.y;
    *reinterpret_cast<__nv_bfloat162*>(h + r * F + i) = __floats2bfloat162_rn(a, c);
}

// the halves layout at streaming sizes: 8 outputs per thread, 16-byte loads and stores (F % 8 == 0)
__global__ void __launch_bounds__(256) silu_mul_halves_vec_kernel(const bf16* __restrict__ gu, bf16* __restrict__ h, int F8,
                                                                  int64_t total8) {
    const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;     // index over [rows][F/8]
    if (t >= total8) return;
    const int64_t r = t / F8;
    const int c = (int)(t - r * F8);
    const uint4 g4 = ld_nc_u128(gu + (r * 2 * F8 + c) * 8);
    const uint4 u4 = ld_nc_u128(gu + (r * 2 * F8 + F8 + c) * 8);
    const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 gte = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[i]));
        const float2 up = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[i]));
        const __nv_bfloat162 y = __floats2bfloat162_rn(gte.x / (1.0f + __expf(-gte.x)) * up.x, gte.y / (1.0f + __expf(-gte.y)) * up.y);
        ow[i] = *reinterpret_cast<const uint32_t*>(&y);
    }
    *reinterpret_cast<uint4*>(h + t * 8) = o;
}

__global__ void add_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ y, int64_t pairs) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= pairs) return;
    const float2 u = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(a)[t]);
    const float2 v = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(b)[t]);
    reinterpret_cast<__nv_bfloat162*>(y)[t] = __floats2bfloat162_rn(u.x + v.x, u.y + v.y);
}

__global__ void embed_kernel(const int64_t* __restrict__ ids, const bf16* __restrict__ table, bf16* __restrict__ y, int D,
                             int vocab) {
    int64_t id = ids[blockIdx.x];
    if (id < 0) id = 0;
    if (id >= vocab) id = vocab - 1;
    const uint4* src = reinterpret_cast<const uint4*>(table + id * D);
    uint4* dst = reinterpret_cast<uint4*>(y + (int64_t)blockIdx.x * D);
    for (int i = threadIdx.x; i < D / 8; i += blockDim.x) dst[i] = src[i];
}

// ---- greedy sampling: ids[r] = argmax_v logits[r][v] (first maximum wins) ----------------------
__global__ void __launch_bounds__(1024) argmax_kernel(const bf16* __restrict__ logits, int64_t* __restrict__ ids, int V) {
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    const bf16* row = logits + (int64_t)blockIdx.x * V;
    float best = -FLT_MAX;
    int bi = 0x7fffffff;
    if ((V & 7) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
        // 8 logits per 16-byte load; a thread's indices still increase, so "first maximum" is kept by '>'
        for (int i8 = threadIdx.x; i8 < V / 8; i8 += 1024) {
            const uint4 u = *reinterpret_cast<const uint4*>(row + (int64_t)i8 * 8);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
                if (f.x > best) { best = f.x; bi = i8 * 8 + 2 * j; }
                if (f.y > best) { best = f.y; bi = i8 * 8 + 2 * j + 1; }
            }
        }
    } else {
        for (int i = threadIdx.x; i < V; i += 1024) {
            const float v = __bfloat162float(row[i]);
            if (v > best) { best = v; bi = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { s_v[threadIdx.x >> 5] = best; s_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = s_v[threadIdx.x];
        bi = s_i[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (threadIdx.x == 0) ids[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

// host side: copies the attention status word (synchronises)
int attn_read_error(unsigned int* out4) {
    NF4_CUDA_TRY(cudaMemcpyFromSymbol(out4, g_attn_error, sizeof(unsigned int) * 4));
    return NF4_OK;
}
int attn_clear_error() {
    const unsigned int zero[4] = {0u, 0u, 0u, 0u};
    NF4_CUDA_TRY(cudaMemcpyToSymbol(g_attn_error, zero, sizeof(zero)));
    return NF4_OK;
}

}  // namespace nf4

using namespace nf4;

extern "C" int nf4_b200_rmsnorm(const void* x, const void* w, void* y, int64_t rows, int64_t D, float eps, void* stream) {
    NF4_REQUIRE(x && w && y, NF4_ERR_ARG, "rmsnorm: null pointer");
    NF4_REQUIRE(rows >= 0 && D > 0 && D % 2 == 0, NF4_ERR_ARG, "rmsnorm: rows=%lld D=%lld (D must be even)", (long long)rows, (long long)D);
    if (rows == 0) return NF4_OK;
    rmsnorm_kernel<<<(unsigned)rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const bf16*>(x), static_cast<const bf16*>(w),
                                                                               static_cast<bf16*>(y), (int)D, eps);
    NF4_CUDA_TRY(cudaGetLastError());
    return NF4_OK;
}

extern "C" int nf4_b200_rope_append(const void* qkv, const int* positions, void* q_out, void* k_cache, void* v_cache,
                                    int64_t B, int Hq, int Hkv, int Dh, int64_t S_max, float theta, void* stream) {
    NF4_REQUIRE(qkv && positions && q_out && k_cache && v_cache, NF4_ERR_ARG, "rope_append: null pointer");
    NF4_REQUIRE(Dh % 2 == 0 && Dh <= 2048 && Hq > 0 && Hkv > 0, NF4_ERR_ARG, "rope_append: bad head geometry");
    NF4_REQUIRE(S_max > 0 && S_max <= 0x7fffffff, NF4_ERR_ARG, "rope_append: S_max=%lld", (long long)S_max);
    if (B == 0) return NF4_OK;
    dim3 grid((unsigned)(Hq + 2 * Hkv), (unsigned)B);
    rope_append_kernel<<<grid, Dh / 2, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf16*>(qkv), positions, static_cast<bf16*>(q_out), static_cast<bf16*>(k_cache),
        static_cast<bf16*>(v_cache), Hq, Hkv, Dh, (int)S_max, theta);
    NF4_CUDA_TRY(cudaGetLastError());
    return NF4_OK;
}

extern "C" int nf4_b200_rope_prefill(const void* qkv, const int* positions, void* q_out, void* k_cache, void* v_cache,
                                     int64_t B, int64_t T, int Hq, int Hkv, int Dh, int64_t S_max, float theta, void* stream) {
    NF4_REQUIRE(qkv && positions && q_out && k_cache && v_cache, NF4_ERR_ARG, "rope_prefill: null pointer");
    NF4_REQUIRE(Dh >= 2 && Dh <= 512 && 256 % (Dh / 2) == 0 && Dh % 2 == 0 && Hq > 0 && Hkv > 0, NF4_ERR_ARG,
                "rope_prefill: head_dim %d (a power of two up to 512)", Dh);
    NF4_REQUIRE(S_max > 0 && S_max <= 0x7fffffff && T >= 0 && T <= 0x7fffffff && B >= 0 && B <= 65535, NF4_ERR_ARG,
                "rope_prefill: B=%lld T=%lld S_max=%lld", (long long)B, (long long)T, (long long)S_max);
    if (B == 0 || T == 0) return NF4_OK;
    dim3 grid((unsigned)T, (unsigned)B);
    rope_prefill_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf16*>(qkv), positions, static_cast<bf16*>(q_out), static_cast<bf16*>(k_cache),
        static_cast<bf16*>(v_cache), (int)T, Hq, Hkv, Dh, (int)S_max, theta);
    NF4_CUDA_TRY(cudaGetLastError());
    return NF4_OK;
}

extern "C" int64_t nf4_b200_attn_decode_workspace_bytes(int64_t B, int Hq, int nsplit) {
    return B * Hq * (int64_t)nsplit * (128 + 2) * 4;
}

// the attention kernels need more dynamic shared memory than the default limit: opt in once per device
static int attn_configure() {
    static bool configured[64] = {false};
    int dev = 0;
    NF4_CUDA_TRY(cudaGetDevice(&dev));
    NF4_REQUIRE(dev < 64, NF4_ERR_LIMIT, "attention: device ordinal %d (at most 64 devices per process)", dev);
    if (configured[dev]) return NF4_OK;
#define NF4_AT_OPT_IN(K) NF4_CUDA_TRY(cudaFuncSetAttribute(K, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM_BYTES))
    NF4_AT_OPT_IN(attn_decode_kernel<1>); NF4_AT_OPT_IN(attn_decode_kernel<2>);
    NF4_AT_OPT_IN(attn_decode_kernel<4>); NF4_AT_OPT_IN(attn_decode_kernel<8>);
    NF4_AT_OPT_IN(attn_fused_kernel<1>); NF4_AT_OPT_IN(attn_fused_kernel<2>);
    NF4_AT_OPT_IN(attn_fused_kernel<4>); NF4_AT_OPT_IN(attn_fused_kernel<8>);
#undef NF4_AT_OPT_IN
    configured[dev] = true;
    return NF4_OK;
}

static int attn_decode_launch(const void* q, const void* k_cache, const void* v_cache, const int* positions, void* out,
                              void* workspace, int64_t B, int Hq, int Hkv, int Dh, int64_t S_max, int nsplit,
                              void* stream) {
    NF4_REQUIRE(q && k_cache && v_cache && positions && out && workspace, NF4_ERR_ARG, "attn_decode: null pointer");
    NF4_REQUIRE(Dh == 128, NF4_ERR_ARG, "attn_decode: head_dim %d (only 128)", Dh);
    NF4_REQUIRE(Hkv > 0 && Hq % Hkv == 0 && nsplit >= 1 && nsplit <= 32, NF4_ERR_ARG, "attn_decode: bad geometry (1 <= nsplit <= 32)");
    NF4_REQUIRE(S_max > 0 && S_max <= 0x7fffffff, NF4_ERR_ARG, "attn_decode: S_max=%lld", (long long)S_max);
    if (B == 0) return NF4_OK;
    const int G = Hq / Hkv;
    if (int rc = attn_configure()) return rc;
    dim3 grid((unsigned)Hkv, (unsigned)B, (unsigned)nsplit);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const float scale = 1.0f / sqrtf((float)Dh);
    const bf16* qq = static_cast<const bf16*>(q);
    const bf16* kk = static_cast<const bf16*>(k_cache);
    const bf16* vv = static_cast<const bf16*>(v_cache);
    float* ws = static_cast<float*>(workspace);
    switch (G) {
        case 1: attn_decode_kernel<1><<<grid, 128, AT_SMEM_BYTES, s>>>(qq, kk, vv, positions, ws, Hq, Hkv, (int)S_max, nsplit, scale); break;
        case 2: attn_decode_kernel<2><<<grid, 128, AT_SMEM_BYTES, s>>>(qq, kk, vv, positions, ws, Hq, Hkv, (int)S_max, nsplit, scale); break;
        case 4: attn_decode_kernel<4><<<grid, 128, AT_SMEM_BYTES, s>>>(qq, kk, vv, positions, ws, Hq, Hkv, (int)S_max, nsplit, scale); break;
        case 8: attn_decode_kernel<8><<<grid, 128, AT_SMEM_BYTES, s>>>(qq, kk, vv, positions, ws, Hq, Hkv, (int)S_max, nsplit, scale); break;
        default:
            set_error("attn_decode: %d query heads per KV head (supported: 1, 2, 4, 8)", G);
            return NF4_ERR_ARG;
    }
    NF4_CUDA_TRY(cudaGetLastError());
    attn_combine_kernel<<<(unsigned)((B * Hq + 3) / 4), 128, 0, s>>>(ws, static_cast<bf16*>(out), nsplit, (int)(B * Hq));
    NF4_CUDA_TRY(cudaGetLastError());
    return NF4_OK;
}

extern "C" int nf4_b200_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int* positions,
                                    void* out, void* workspace, int64_t B, int Hq, int Hkv, int Dh, int64_t S_max,
                                    int nsplit, void* stream) {
    return attn_decode_launch(q, k_cache, v_cache, positions, out, workspace, B, Hq, Hkv, Dh, S_max, nsplit, stream);
}

// ---- attention without a caller-provided workspace ---------------------------------------------
// Scratch for the per-split partial results lives in this fixed device array instead of a buffer
// the caller allocates.  It is sized for the largest decode shape this library targets:
// 16 batch rows x 64 query heads x 8 sequence splits.  Every GPU that loads the library carries
// these 4,259,840 bytes until the process exits.
constexpr int64_t ATTN_STATIC_WS_BYTES = 16ll * 64 * 8 * (128 + 2) * 4;
static __device__ __align__(256) unsigned char g_attn_static_ws[ATTN_STATIC_WS_BYTES];

// In host code `g_attn_static_ws` is only a handle for the runtime, not an address a kernel can
// use; the device address has to be asked for, once per device, while that device is current.
static int attn_static_ws_ptr(void** out) {
    static void* ptrs[64] = {nullptr};
    int dev = 0;
    NF4_CUDA_TRY(cudaGetDevice(&dev));
    NF4_REQUIRE(dev >= 0 && dev < 64, NF4_ERR_LIMIT, "attn_decode_static: device ordinal %d above 63", dev);
    if (ptrs[dev] == nullptr) {
        void* p = nullptr;
        NF4_CUDA_TRY(cudaGetSymbolAddress(&p, g_attn_static_ws));
        NF4_REQUIRE(p != nullptr, NF4_ERR_CUDA, "attn_decode_static: cudaGetSymbolAddress returned a null address");
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return NF4_OK;
}

extern "C" int64_t nf4_b200_attn_decode_static_max_bytes(void) { return ATTN_STATIC_WS_BYTES; }

extern "C" int nf4_b200_attn_decode_static(const void* q, const void* k_cache, const void* v_cache, const int* positions,
                                           void* out, int64_t B, int Hq, int Hkv, int Dh, int64_t S_max, int nsplit,
                                           void* stream) {
    NF4_REQUIRE(B >= 0 && Hq > 0 && nsplit >= 1, NF4_ERR_ARG, "attn_decode_static: bad extents");
    const int64_t need = nf4_b200_attn_decode_workspace_bytes(B, Hq, nsplit);
    NF4_REQUIRE(need <= ATTN_STATIC_WS_BYTES, NF4_ERR_LIMIT,
                "attn_decode_static: B=%lld x Hq=%d x nsplit=%d needs %lld bytes of scratch, the built-in array holds %lld "
                "(16 x 64 x 8); use nf4_b200_attn_decode with your own workspace",
                (long long)B, Hq, nsplit, (long long)need, (long long)ATTN_STATIC_WS_BYTES);
    void* ws = nullptr;
    if (int rc = attn_static_ws_ptr(&ws)) return rc;
    return attn_decode_launch(q, k_cache, v_cache, positions, out, ws, B, Hq, Hkv, Dh, S_max, nsplit, stream);
}

extern "C" int nf4_b200_attn_decode_fused(const void* qkv, const int* positions, void* k_cache, void* v_cache, void* out,
                                          void* workspace, unsigned int* counters, int64_t B, int Hq, int Hkv, int Dh,
                                          int64_t S_max, int nsplit, float theta, int flags, void* stream) {
    NF4_REQUIRE(qkv && positions && k_cache && v_cache && out && workspace && counters, NF4_ERR_ARG, "attn_decode_fused: null pointer");
    NF4_REQUIRE(Dh == 128, NF4_ERR_ARG, "attn_decode_fused: head_dim %d (only 128)", Dh);
    NF4_REQUIRE(Hkv > 0 && Hq % Hkv == 0 && nsplit >= 1 && nsplit <= 32, NF4_ERR_ARG, "attn_decode_fused: bad geometry (1 <= nsplit <= 32)");
    NF4_REQUIRE(S_max > 0 && S_max <= 0x7fffffff, NF4_ERR_ARG, "attn_decode_fused: S_max=%lld", (long long)S_max);
    if (B == 0) return NF4_OK;
    const int G = Hq / Hkv;
    NF4_REQUIRE(G == 1 || G == 2 || G == 4 || G == 8, NF4_ERR_ARG, "attn_decode_fused: %d query heads per KV head", G);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)Hkv, (unsigned)B, (unsigned)nsplit);
    cfg.blockDim = dim3(128);
    if (int rc = attn_configure()) return rc;
    cfg.dynamicSmemBytes = AT_SMEM_BYTES;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & 1) ? 1 : 0;
    const float scale = 1.0f / sqrtf((float)Dh);
    const bf16* a0 = static_cast<const bf16*>(qkv);
    bf16* a2 = static_cast<bf16*>(k_cache);
    bf16* a3 = static_cast<bf16*>(v_cache);
    bf16* a4 = static_cast<bf16*>(out);
    float* a5 = static_cast<float*>(workspace);
    const int smax = (int)S_max;
    switch (G) {
        case 1: NF4_CUDA_TRY(cudaLaunchKernelEx(&cfg, attn_fused_kernel<1>, a0, positions, a2, a3, a4, a5, counters, Hq, Hkv, smax, nsplit, scale, theta)); break;
        case 2: NF4_CUDA_TRY(cudaLaunchKernelEx(&cfg, attn_fused_kernel<2>, a0, positions, a2, a3, a4, a5, counters, Hq, Hkv, smax, nsplit, scale, theta)); break;
        case 4: NF4_CUDA_TRY(cudaLaunchKernelEx(&cfg, attn_fused_kernel<4>, a0, positions, a2, a3, a4, a5, counters, Hq, Hkv, smax, nsplit, scale, theta)); break;
        default: NF4_CUDA_TRY(cudaLaunchKernelEx(&cfg, attn_fused_kernel<8>, a0, positions, a2, a3, a4, a5, counters, Hq, Hkv, smax, nsplit, scale, theta)); break;
    }
    return NF4_OK;
}

extern "C" int nf4_b200_silu_mul(const void* gate_up, void* h, int64_t rows, int64_t F, int interleaved, void* stream) {
    NF4_REQUIRE(gate_up && h, NF4_ERR_ARG, "silu_mul: null pointer");
    NF4_REQUIRE(rows >= 0 && F > 0 && F % 2 == 0, NF4_ERR_ARG, "silu_mul: bad extents");
    const int64_t pairs = rows * (F / 2);
    if (pairs == 0) return NF4_OK;
    if (!interleaved && F % 8 == 0 && rows * F >= (1 << 20) && reinterpret_cast<uintptr_t>(gate_up) % 16 == 0 &&
        reinterpret_cast<uintptr_t>(h) % 16 == 0) {
        const int64_t total8 = rows * (F / 8);
        silu_mul_halves_vec_kernel<<<(unsigned)((total8 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const bf16*>(gate_up), static_cast<bf16*>(h), (int)(F / 8), total8);
        NF4_CUDA_TRY(cudaGetLastError());
        return NF4_OK;
    }
    silu_mul_kernel<<<(unsigned)((pairs + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf16*>(gate_up), static_cast<bf16*>(h), (int)F, pairs, interleaved);
    NF4_CUDA_TRY(cudaGetLastError());
    return NF4_OK;
}

extern "C" int nf4_b200_add(const void* a, const void* b, void* y, int64_t numel, void* stream) {
    NF4_REQUIRE(a && b && y, NF4_ERR_ARG, "add: null pointer");
    NF4_REQUIRE(numel >= 0 && numel % 2 == 0, NF4_ERR_ARG, "add: numel must be even");
    if (numel == 0) return NF4_OK;
    add_kernel<<<(unsigned)((numel / 2 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf16*>(a), static_cast<const bf16*>(b), static_cast<bf16*>(y), numel / 2);
    NF4_CUDA_TRY(cudaGetLastError());
    return NF4_OK;
}

extern "C" int nf4_b200_embed(const int64_t* ids, const void* table, void* y, int64_t rows, int64_t D, int64_t vocab,
                              void* stream) {
    NF4_REQUIRE(ids && table && y, NF4_ERR_ARG, "embed: null pointer");
    NF4_REQUIRE(D > 0 && D % 8 == 0 && vocab > 0, NF4_ERR_ARG, "embed: D must be a multiple of 8");
    if (rows == 0) return NF4_OK;
    embed_kernel<<<(unsigned)rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(ids, static_cast<const bf16*>(table), static_cast<bf16*>(y),
                                                                              (int)D, (int)vocab);
    NF4_CUDA_TRY(cudaGetLastError());
    return NF4_OK;
}

extern "C" int nf4_b200_argmax(const void* logits, int64_t* ids, int64_t rows, int64_t V, void* stream) {
    NF4_REQUIRE(logits && ids, NF4_ERR_ARG, "argmax: null pointer");
    NF4_REQUIRE(V > 0 && V < (1ll << 31), NF4_ERR_ARG, "argmax: bad vocabulary size");
    if (rows == 0) return NF4_OK;
    argmax_kernel<<<(unsigned)rows, 1024, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const bf16*>(logits), ids, (int)V);
    NF4_CUDA_TRY(cudaGetLastError());
    return NF4_OK;
}
