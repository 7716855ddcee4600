// One-shot all-reduce of the row-parallel projections' partial outputs over NVLink peer memory.
//
// Tensor-parallel decode sums, after the attention-output and the MLP-down projection, one small
// [M, d_model] bf16 tile per rank (256 KB at 16 x 8192).  A library all-reduce of that size is bound by
// its fixed latency; this kernel does the exchange in one launch with plain peer stores:
//
//   every rank owns a "symmetric" buffer that all ranks have mapped (the caller passes the `world`
//   base addresses as seen from this rank):   flags | per-block epochs | data[2 sets][world sources]
//
//   block b of rank r:   1. copies chunk b of its partial tile into slot (set, r) of EVERY rank's buffer
//                           (16-byte stores; set = epoch & 1, so a fast rank never overwrites what a slow
//                           rank still reads),
//                        2. publishes that with a release store of the epoch to flag (set, b, r) of every rank,
//                        3. waits -- bounded -- until its own flags (set, b, 0..world-1) carry the epoch,
//                        4. adds the `world` chunks in rank order in fp32 (+ an optional residual) and writes
//                           bf16: every rank computes the same bits.
//
// Block b only ever needs chunk b of every rank, so there is no grid-wide step.  The epoch of a block is a
// counter in device memory that the block itself advances, which makes the kernel replayable from a CUDA
// graph.  No loads from peer memory, no multicast, no TMA: remote data is always WRITTEN into the consumer's
// own memory first.  A wait that runs out records code 10 in the status word (nf4_b200_device_error) and the
// block finishes with whatever has arrived -- it never spins forever.
//
// `nf4_b200_tp_allreduce_emulated` runs all ranks of one exchange as ONE cooperative launch on one GPU
// (blockIdx.y = rank), so the protocol can be tested without several GPUs and without kernels that wait
// on one another in separate launches.
#include <cooperative_groups.h>

#include "nf4_common.cuh"

namespace nf4 {

typedef __nv_bfloat16 bf16;

constexpr int AR_MAX_WORLD = 8;
constexpr int AR_MAX_BLOCKS = 64;
constexpr int AR_THREADS = 256;
constexpr int64_t AR_FLAGS_BYTES = 2 * AR_MAX_BLOCKS * AR_MAX_WORLD * 4;   // [set][block][source]
constexpr int64_t AR_EPOCH_BYTES = AR_MAX_BLOCKS * 4;                     // [block], local use only
constexpr int64_t AR_DATA_OFFSET = 8192;                                  // flags + epochs, padded
constexpr unsigned long long AR_WAIT_LIMIT_NS = 500ull * 1000 * 1000;     // 0.5 s per wait

__device__ unsigned int g_ar_error[4];   // [0] code (10 = a flag wait ran out), [1] block, [2] source rank, [3] count

struct ArParams {
    const bf16* partial[AR_MAX_WORLD];    // [rank] (only [0] outside of the emulation)
    const bf16* residual[AR_MAX_WORLD];
    bf16* y[AR_MAX_WORLD];
    uint8_t* bufs[AR_MAX_WORLD];          // base of every rank's buffer, indexed by rank
    int rank, world;
    int64_t numel;                        // bf16 elements of the tile (multiple of 8)
    int64_t chunk;                        // elements per block (multiple of 8)
    int64_t slot_bytes;                   // bytes between slots
    int emulated;                         // blockIdx.y is the rank
    int pdl;                              // launched with programmatic stream serialization
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ar_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(AR_THREADS) tp_allreduce_kernel(const __grid_constant__ ArParams p) {
    // Programmatic dependent launch: the next kernel of the stream (a GEMV that starts by streaming weights) may
    // become resident now; this kernel itself may have started while its predecessor (the GEMV that writes
    // `partial`) was still running and waits for it below, before it reads anything the predecessor wrote.
    if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int b = blockIdx.x;
    const int rank = p.emulated ? (int)blockIdx.y : p.rank;
    const int slot = p.emulated ? rank : 0;
    const int tid = threadIdx.x;
    uint8_t* const mine = p.bufs[rank];
    __shared__ uint32_t s_epoch;
    if (tid == 0) {
        uint32_t* ep = reinterpret_cast<uint32_t*>(mine + AR_FLAGS_BYTES) + b;
        const uint32_t e = *ep + 1u;
        *ep = e;
        s_epoch = e;
    }
    __syncthreads();
    if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t epoch = s_epoch;
    const int set = (int)(epoch & 1u);
    const int64_t e0 = (int64_t)b * p.chunk;
    const int64_t e1 = min(p.numel, e0 + p.chunk);
    const int64_t nvec = e1 > e0 ? (e1 - e0) / 8 : 0;      // 16-byte vectors of this block's chunk

    // 1. my chunk -> slot (set, rank) of every rank (the own buffer included), starting with the next rank
    const uint4* src = reinterpret_cast<const uint4*>(p.partial[slot] + e0);
    for (int64_t v = tid; v < nvec; v += AR_THREADS) {
        const uint4 val = src[v];
        for (int k = 1; k <= p.world; ++k) {
            const int peer = (rank + k) % p.world;
            uint4* dst = reinterpret_cast<uint4*>(p.bufs[peer] + AR_DATA_OFFSET + (int64_t)(set * AR_MAX_WORLD + rank) * p.slot_bytes) + (e0 / 8) + v;
            *dst = val;
        }
    }
    __threadfence_system();
    __syncthreads();
    // 2. publish, 3. wait for every source (thread t handles rank t)
    if (tid < p.world) {
        uint32_t* remote = reinterpret_cast<uint32_t*>(p.bufs[tid]) + ((int64_t)set * AR_MAX_BLOCKS + b) * AR_MAX_WORLD + rank;
        st_release_sys(remote, epoch);
        const uint32_t* local = reinterpret_cast<const uint32_t*>(mine) + ((int64_t)set * AR_MAX_BLOCKS + b) * AR_MAX_WORLD + tid;
        bool seen = false;
        for (int spin = 0; spin < 4096 && !seen; ++spin) seen = ld_acquire_sys(local) == epoch;
        if (!seen) {
            const unsigned long long t0 = ar_ns();
            while (!seen) {
                for (int spin = 0; spin < 256 && !seen; ++spin) seen = ld_acquire_sys(local) == epoch;
                if (!seen && ar_ns() - t0 > AR_WAIT_LIMIT_NS) {
                    if (atomicCAS(&g_ar_error[0], 0u, 10u) == 0u) {
                        g_ar_error[1] = (unsigned)b;
                        g_ar_error[2] = (unsigned)tid;
                    }
                    atomicAdd(&g_ar_error[3], 1u);
                    break;
                }
            }
        }
    }
    __syncthreads();
    // 4. sum the chunks in rank order (fp32), add the residual, round once
    const uint4* res = p.residual[slot] ? reinterpret_cast<const uint4*>(p.residual[slot] + e0) : nullptr;
    uint4* out = reinterpret_cast<uint4*>(p.y[slot] + e0);
    for (int64_t v = tid; v < nvec; v += AR_THREADS) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int r = 0; r < p.world; ++r) {
            const uint4* s = reinterpret_cast<const uint4*>(mine + AR_DATA_OFFSET + (int64_t)(set * AR_MAX_WORLD + r) * p.slot_bytes) + (e0 / 8) + v;
            const uint4 val = __ldcg(s);      // written by a peer: read from L2, never from a stale L1 line
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&val);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h[j]);
                acc[2 * j] += f.x;
                acc[2 * j + 1] += f.y;
            }
        }
        if (res) {
            const uint4 val = res[v];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&val);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h[j]);
                acc[2 * j] += f.x;
                acc[2 * j + 1] += f.y;
            }
        }
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        out[v] = o;
    }
}

// host side: copies the all-reduce status word (synchronises)
int ar_read_error(unsigned int* out4) {
    NF4_CUDA_TRY(cudaMemcpyFromSymbol(out4, g_ar_error, sizeof(unsigned int) * 4));
    return NF4_OK;
}
int ar_clear_error() {
    const unsigned int zero[4] = {0u, 0u, 0u, 0u};
    NF4_CUDA_TRY(cudaMemcpyToSymbol(g_ar_error, zero, sizeof(zero)));
    return NF4_OK;
}

static int ar_plan(int64_t numel, int world, int64_t buffer_bytes, ArParams* p, int* blocks_out) {
    NF4_REQUIRE(world >= 1 && world <= AR_MAX_WORLD, NF4_ERR_LIMIT, "tp_allreduce: world %d outside [1, %d]", world, AR_MAX_WORLD);
    NF4_REQUIRE(numel > 0 && numel % 8 == 0, NF4_ERR_ARG, "tp_allreduce: numel %lld must be a positive multiple of 8", (long long)numel);
    const int64_t slot = (numel * 2 + 255) / 256 * 256;
    NF4_REQUIRE(buffer_bytes >= AR_DATA_OFFSET + 2 * AR_MAX_WORLD * slot, NF4_ERR_WORKSPACE,
                "tp_allreduce: buffers of %lld bytes, need %lld (nf4_b200_tp_allreduce_buffer_bytes)", (long long)buffer_bytes,
                (long long)(AR_DATA_OFFSET + 2 * AR_MAX_WORLD * slot));
    // the slot pitch is fixed by the buffer size, not by this call's numel, so calls of different sizes can share a buffer
    p->slot_bytes = ((buffer_bytes - AR_DATA_OFFSET) / (2 * AR_MAX_WORLD)) / 256 * 256;
    int64_t blocks = (numel / 8 + 511) / 512;            // >= 512 vectors (8 KB) per block
    if (blocks > AR_MAX_BLOCKS) blocks = AR_MAX_BLOCKS;
    if (blocks < 1) blocks = 1;
    p->chunk = ((numel / 8 + blocks - 1) / blocks) * 8;
    p->numel = numel;
    p->world = world;
    *blocks_out = (int)((numel + p->chunk - 1) / p->chunk);
    return NF4_OK;
}

}  // namespace nf4

using namespace nf4;

extern "C" int64_t nf4_b200_tp_allreduce_buffer_bytes(int64_t max_numel) {
    if (max_numel < 8) max_numel = 8;
    const int64_t slot = (max_numel * 2 + 255) / 256 * 256;
    return AR_DATA_OFFSET + 2 * AR_MAX_WORLD * slot;
}

extern "C" int nf4_b200_tp_allreduce(const void* partial, const void* residual, void* y, int64_t numel,
                                     const uint64_t* host_buffer_ptrs, int64_t buffer_bytes, int rank, int world, int flags,
                                     void* stream) {
    NF4_REQUIRE(partial && y && host_buffer_ptrs, NF4_ERR_ARG, "tp_allreduce: null pointer");
    NF4_REQUIRE(rank >= 0 && rank < world, NF4_ERR_ARG, "tp_allreduce: rank %d of %d", rank, world);
    NF4_REQUIRE(reinterpret_cast<uintptr_t>(partial) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0 &&
                reinterpret_cast<uintptr_t>(residual) % 16 == 0, NF4_ERR_ALIGN, "tp_allreduce: tensors must be 16-byte aligned");
    ArParams p = {};
    int blocks = 0;
    if (int rc = ar_plan(numel, world, buffer_bytes, &p, &blocks)) return rc;
    if (int rc = check_device()) return rc;
    for (int r = 0; r < world; ++r) {
        NF4_REQUIRE(host_buffer_ptrs[r] != 0 && host_buffer_ptrs[r] % 256 == 0, NF4_ERR_ALIGN, "tp_allreduce: buffer %d is null or not 256-byte aligned", r);
        p.bufs[r] = reinterpret_cast<uint8_t*>(host_buffer_ptrs[r]);
    }
    p.partial[0] = static_cast<const bf16*>(partial);
    p.residual[0] = static_cast<const bf16*>(residual);
    p.y[0] = static_cast<bf16*>(y);
    p.rank = rank;
    p.emulated = 0;
    p.pdl = flags & 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(AR_THREADS);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl ? 1 : 0;
    NF4_CUDA_TRY(cudaLaunchKernelEx(&cfg, tp_allreduce_kernel, p));
    return NF4_OK;
}

extern "C" int nf4_b200_tp_allreduce_emulated(const uint64_t* host_partial_ptrs, const uint64_t* host_residual_ptrs,
                                              const uint64_t* host_y_ptrs, int64_t numel, const uint64_t* host_buffer_ptrs,
                                              int64_t buffer_bytes, int world, void* stream) {
    NF4_REQUIRE(host_partial_ptrs && host_y_ptrs && host_buffer_ptrs, NF4_ERR_ARG, "tp_allreduce_emulated: null pointer");
    ArParams p = {};
    int blocks = 0;
    if (int rc = ar_plan(numel, world, buffer_bytes, &p, &blocks)) return rc;
    if (int rc = check_device()) return rc;
    int per_sm = 0;
    NF4_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tp_allreduce_kernel, AR_THREADS, 0));
    NF4_REQUIRE(blocks * world <= sm_count() * per_sm, NF4_ERR_LIMIT,
                "tp_allreduce_emulated: %d blocks x %d ranks do not fit on the device at once", blocks, world);
    for (int r = 0; r < world; ++r) {
        NF4_REQUIRE(host_buffer_ptrs[r] % 256 == 0 && host_partial_ptrs[r] % 16 == 0 && host_y_ptrs[r] % 16 == 0, NF4_ERR_ALIGN,
                    "tp_allreduce_emulated: rank %d has a misaligned pointer", r);
        p.bufs[r] = reinterpret_cast<uint8_t*>(host_buffer_ptrs[r]);
        p.partial[r] = reinterpret_cast<const bf16*>(host_partial_ptrs[r]);
        p.residual[r] = host_residual_ptrs ? reinterpret_cast<const bf16*>(host_residual_ptrs[r]) : nullptr;
        p.y[r] = reinterpret_cast<bf16*>(host_y_ptrs[r]);
    }
    p.rank = 0;
    p.emulated = 1;
    // the blocks of different ranks wait on one another: a cooperative launch guarantees they are all resident
    void* args[] = {&p};
    NF4_CUDA_TRY(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(tp_allreduce_kernel), dim3((unsigned)blocks, (unsigned)world),
                                             dim3(AR_THREADS), args, 0, static_cast<cudaStream_t>(stream)));
    return NF4_OK;
}
