/*
 * C ABI of libnf4_b200.so -- the sm_100a kernels behind Thunder's NF4 quantized-linear path.
 *
 * Every entry point replaces one call the reference makes into the bitsandbytes package
 * (the reference has no FFI of its own: thunder/transforms/quantization.py is pure Python
 * and reaches CUDA only through those calls).  All pointers are DEVICE pointers unless a
 * parameter is named host_*; `stream` is a cudaStream_t passed as void* (NULL = the legacy
 * default stream).  Functions return 0 on success or an NF4_ERR_* code, never throw, never
 * synchronise the device and never allocate device memory (the caller owns every buffer), so
 * they may be called while a stream is being captured into a CUDA graph.
 * nf4_b200_last_error() gives the message of the last failure on the calling thread.
 *
 * Tensor contract (thunder/transforms/quantization.py:86-101): a weight W[N,K] (row-major,
 * numel = N*K) is stored as
 *     packed  uint8 [ceil(numel/2)]     byte j = (index[2j] << 4) | index[2j+1]
 *     absmax  fp32  [ceil(numel/blocksize)]   one scale per `blocksize` consecutive elements
 *     code16  fp32  [16]                the level table (the op's `quant_map` argument)
 */
#ifndef NF4_B200_H
#define NF4_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    NF4_OK = 0,
    NF4_ERR_ARG = 1,       /* null pointer, negative extent, unsupported dtype/blocksize */
    NF4_ERR_ALIGN = 2,     /* a pointer breaks the documented alignment */
    NF4_ERR_WORKSPACE = 3, /* workspace too small */
    NF4_ERR_CUDA = 4,      /* a CUDA runtime call failed (message holds cudaGetErrorString) */
    NF4_ERR_ARCH = 5,      /* the current device is not compute capability 10.x */
    NF4_ERR_LIMIT = 6      /* a size exceeds a documented maximum */
};

/* element types of weights / activations / outputs */
enum { NF4_F32 = 0, NF4_F16 = 1, NF4_BF16 = 2 };

int nf4_b200_version(void);

/* Copies the calling thread's last error message (NUL terminated) into buf; returns its length. */
int nf4_b200_last_error(char* buf, int buflen);

/*
 * Blockwise NF4 quantization.  Replaces bitsandbytes.functional.quantize_4bit(w, quant_type="nf4")
 * as called at thunder/transforms/quantization.py:63.
 *   w       [numel] of w_dtype, contiguous
 *   packed  [ceil(numel/2)] out, absmax [ceil(numel/blocksize)] out
 * blocksize: power of two, 64..4096.  Results are bit-exact with the CPU oracle: fp32 absmax,
 * IEEE division, nearest level with the lower index winning a tie, all-zero block -> level 0.0.
 */
int nf4_b200_quantize(const void* w, int64_t numel, int w_dtype, int blocksize, const float* code16,
                      uint8_t* packed, float* absmax, void* stream);

/*
 * Blockwise dequantization: out[i] = round_to(out_dtype, code16[index[i]] * absmax[i / blocksize]).
 * Replaces the dequantize step inside bitsandbytes.matmul_4bit (thunder/transforms/quantization.py:39)
 * and bitsandbytes.functional.dequantize_4bit.
 */
int nf4_b200_dequantize(const uint8_t* packed, const float* absmax, const float* code16, int64_t numel,
                        int blocksize, void* out, int out_dtype, void* stream);

/*
 * y[M,N] = x[M,K] . dequant(W[N,K])^T (+ bias[N]).  Replaces bitsandbytes.matmul_4bit(x, qweight.t(),
 * bias=, quant_state=) as called by bnb_matmul_nf4_impl (thunder/transforms/quantization.py:34-39).
 *   x, y, bias  of `dtype` (x row stride = K, y row stride = N); bias may be NULL
 *   workspace   device scratch of at least nf4_b200_linear_workspace_bytes(M, N, K, dtype) bytes
 *               (may be NULL when that is 0).  It must be zero-filled once before its first use; every
 *               call leaves it ready for the next one.  One workspace serves one stream at a time.
 *               Without it the result is the same sums computed by fewer thread blocks.
 * Dispatch: M <= 16 with K % 64 == 0, blocksize 64 and 16-bit dtype -> fused dequant-GEMV
 * (weights streamed once); larger M in bf16 -> tensor-core dequant-GEMM, K split over thread blocks when
 * the weight has few 128-row tiles; larger M in fp16 -> the fused GEMV once per slab of 16 rows; anything
 * else (fp32, ragged K, other blocksizes) -> a generic kernel.  fp32 accumulation everywhere.
 */
int nf4_b200_linear(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                    const float* code16, int64_t N, int blocksize, const void* bias, void* y, int dtype,
                    void* workspace, int64_t workspace_bytes, void* stream);

int64_t nf4_b200_linear_workspace_bytes(int64_t M, int64_t N, int64_t K, int dtype);

/* Which kernel family the calling thread's last nf4_b200_linear call chose (0 before the first call); for tests
 * and diagnosis.  No counterpart in the reference. */
enum { NF4_PATH_GEMV = 1, NF4_PATH_GEMM = 2, NF4_PATH_GEMV_SLABS = 3, NF4_PATH_GENERIC = 4 };
int nf4_b200_last_linear_path(void);

/* The three kernels behind nf4_b200_linear, callable directly (same argument meaning). */
int nf4_b200_gemv(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                  const float* code16, int64_t N, const void* bias, void* y, int dtype, void* stream);
int nf4_b200_gemm(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                  const float* code16, int64_t N, const void* bias, void* y, int dtype, void* workspace,
                  int64_t workspace_bytes, void* stream);
int nf4_b200_linear_generic(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                            const float* code16, int64_t N, int blocksize, const void* bias, void* y,
                            int dtype, void* stream);
/* Scratch nf4_b200_gemm / nf4_b200_gemm_decode can use for this shape to split K (0: no split planned). */
int64_t nf4_b200_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K);

/*
 * The tensor-core kernel with a decode step's epilogues (bf16 only): y = x . dequant(W)^T + residual
 * (epilogue 0; residual [M,N] may be NULL or alias y), or, with weight rows stored as (gate_i, up_i)
 * pairs, y[M, N/2] = silu(gate) * up (epilogue 1; both sums rounded to bf16 first).  The batched
 * counterpart of nf4_b200_gemv_decode for batches beyond the GEMV's 16 rows; no counterpart in the reference.
 * workspace as for nf4_b200_linear (nf4_b200_gemm_workspace_bytes); flags bit 0: programmatic dependent
 * launch (the weights of the first K blocks are fetched while the upstream kernel drains).
 */
int nf4_b200_gemm_decode(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                         const float* code16, int64_t N, const void* residual, void* y, int epilogue,
                         void* workspace, int64_t workspace_bytes, int flags, void* stream);

/*
 * Double quantization of absmax: 8-bit indices into a sorted 256-entry table, one fp32 scale per 256
 * values, one fp32 offset (device scalar).  The reference leaves this as a TODO
 * (thunder/transforms/quantization.py:84, 120); results are bit-exact with this library's CPU oracle.
 *   absmax' = fma(code256[absmax_u8[i]], scale2[i / 256], *offset)
 * nf4_b200_linear_dq (blocksize 64): up to 16 activation rows in bf16 with K a multiple of 1024 run the fused
 * dequant-GEMV with the 8-bit absmax expanded inside the kernel (the weight streams as 0.5 + 1/64 + 1/4096
 * bytes per element and `workspace` is not touched); every other case expands absmax into `workspace`
 * (nf4_b200_linear_dq_workspace_bytes(N, K) bytes) and then runs nf4_b200_linear on it -- for the tensor-core
 * GEMM that pass is a few per cent of the multiplication.
 */
int nf4_b200_dq_quantize(const float* absmax, int64_t nblocks, const float* code256, uint8_t* absmax_u8, float* scale2,
                         float* offset, void* stream);
int nf4_b200_dq_dequantize(const uint8_t* absmax_u8, const float* scale2, const float* offset, const float* code256,
                           int64_t nblocks, float* absmax, void* stream);
int64_t nf4_b200_linear_dq_workspace_bytes(int64_t N, int64_t K);
int nf4_b200_linear_dq(const void* x, int64_t M, int64_t K, const uint8_t* packed, const uint8_t* absmax_u8,
                       const float* scale2, const float* offset, const float* code256, const float* code16, int64_t N,
                       const void* bias, void* y, int dtype, void* workspace, int64_t workspace_bytes, void* stream);

/*
 * nf4_b200_gemv with one more epilogue term: y = x . dequant(W)^T + bias + residual, residual [M,N]
 * of `dtype` (may be NULL, may alias y).  The reference has no fused form; it is what a decode step
 * needs after the attention-output and MLP-down projections (thunder/tests/llama2_model.py:187-190).
 */
int nf4_b200_gemv_fused(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                        const float* code16, int64_t N, const void* bias, const void* residual, void* y, int dtype,
                        void* stream);

/*
 * The decode-step form of the fused GEMV (bf16): y = prologue(x) . dequant(W)^T + residual, where the
 * prologue runs on the activations while they sit in shared memory:
 *   prologue 0: none;  1: x <- x * rsqrt(mean(x^2) + eps) * norm_w (RMSNorm, norm_w [K]);
 *   2: x is [M, 2K] = [gate | up] and x <- silu(gate) * up (SwiGLU).
 * epilogue 0: y [M, N];  1: the weight's rows are (gate_i, up_i) pairs (row 2i, row 2i+1) and
 *   y [M, N/2] = silu(x.gate_i) * (x.up_i), both sums rounded to bf16 first (no residual);
 *   2: the same with the weight stored as [gate rows; up rows] (row i and row N/2 + i; N % 16 == 0) --
 *   the layout of two separately quantized matrices placed back to back in memory.
 * flags bit 0: launch with programmatic stream serialization (the kernel starts streaming weights
 * while the previous kernel of the stream is finishing and waits for it before touching x, residual
 * or y; the previous and next kernels must come from this library).  Returns NF4_ERR_LIMIT when the
 * prologue's activations do not fit in shared memory (caller runs the separate kernels instead).
 * No counterpart in the reference: it folds the ops between two linears of
 * thunder/tests/llama2_model.py:142-190 into the second linear.
 */
int nf4_b200_gemv_decode_fits(int64_t M, int64_t N, int64_t K, int prologue);   /* 1 if the call below would fit */
int nf4_b200_gemv_decode(const void* x, int64_t M, int64_t K, const uint8_t* packed, const float* absmax,
                         const float* code16, int64_t N, const void* residual, void* y, int prologue,
                         const void* norm_w, float eps, int epilogue, int flags, void* stream);
/*
 * Optional hint for the NEXT nf4_b200_gemv_decode call made by this host thread (that call consumes it):
 * the weight (packed, absmax, N, K) of the launch that will follow it on the same stream.  Each thread
 * block of the hinted call pulls the head of its share of that weight into L2 once its own loads are in
 * flight, which keeps HBM busy across the kernel boundary.  Purely a prefetch: results do not change, and
 * a hint for a weight that is not read next only wastes bandwidth -- but the hinted buffers must be live
 * device memory of those extents when the hinted call runs (the prefetch touches them).  NULL pointers
 * clear a pending hint.  No counterpart in the reference.
 */
int nf4_b200_gemv_decode_next_weight(const uint8_t* packed, const float* absmax, int64_t N, int64_t K);


/*
 * Decode-step glue kernels (bf16 tensors, fp32 arithmetic).  In the reference these ops are lowered
 * by Thunder's executors from the model's trace (RMSNorm, rotary embedding, attention, SwiGLU:
 * thunder/tests/llama2_model.py:20-40, 57-126, 142-190); here they are single launches so that one
 * decode step of a Llama-shaped model is a short, capturable chain around the NF4 linears.
 */
/* y[r,:] = x[r,:] * rsqrt(mean(x[r,:]^2) + eps) * w[:] */
int nf4_b200_rmsnorm(const void* x, const void* w, void* y, int64_t rows, int64_t D, float eps, void* stream);
/* Rotary embedding (interleaved pairs, base theta) of the q and k parts of qkv [B, (Hq+2*Hkv)*Dh] at
 * positions[B]; q goes to q_out [B, Hq*Dh], rotated k and v go to the caches [B, Hkv, S_max, Dh]. */
int nf4_b200_rope_append(const void* qkv, const int* positions, void* q_out, void* k_cache, void* v_cache,
                         int64_t B, int Hq, int Hkv, int Dh, int64_t S_max, float theta, void* stream);
/* The same for a whole prompt (prefill): qkv [B, T, (Hq+2*Hkv)*Dh], positions[T] shared by the B sequences
 * (the model's input_pos, thunder/tests/llama2_model.py:142-190 indexes its rotary tables with it); rotated q
 * goes out in attention layout q_out [B, Hq, T, Dh], rotated k and v go to cache rows positions[t].  Dh a power of
 * two up to 512.  A position outside [0, S_max) writes no cache row and records code 9. */
int nf4_b200_rope_prefill(const void* qkv, const int* positions, void* q_out, void* k_cache, void* v_cache,
                          int64_t B, int64_t T, int Hq, int Hkv, int Dh, int64_t S_max, float theta, void* stream);
/* Single-query grouped attention over cache positions [0, positions[b]]; out [B, Hq*Dh].  Dh = 128.
 * workspace: nf4_b200_attn_decode_workspace_bytes(B, Hq, nsplit) bytes.
 * In all kernels below a positions[b] outside [0, S_max) touches no cache row: that sequence writes
 * nothing, attends to nothing (its output is zero) and code 9 is recorded in nf4_b200_device_error. */
int64_t nf4_b200_attn_decode_workspace_bytes(int64_t B, int Hq, int nsplit);
int nf4_b200_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int* positions, void* out,
                         void* workspace, int64_t B, int Hq, int Hkv, int Dh, int64_t S_max, int nsplit, void* stream);
/* nf4_b200_rope_append + nf4_b200_attn_decode in ONE launch: reads qkv [B, (Hq+2*Hkv)*Dh], rotates q and
 * the new k at positions[B], appends k, v to the caches and attends over [0, positions[b]].  `counters`:
 * B*Hkv unsigned ints that must be zero before the first call (the kernel leaves them zero).  flags bit
 * 0: programmatic dependent launch (see nf4_b200_gemv_decode); with it the kernel reads `positions` before
 * it waits for its predecessor, so positions must hold their final values before the PRECEDING launch on
 * the stream starts (update them after the attention launches of a step, not between the QKV projection
 * and the attention).  No counterpart in the reference. */
int nf4_b200_attn_decode_fused(const void* qkv, const int* positions, void* k_cache, void* v_cache, void* out,
                               void* workspace, unsigned int* counters, int64_t B, int Hq, int Hkv, int Dh,
                               int64_t S_max, int nsplit, float theta, int flags, void* stream);
/*
 * nf4_b200_attn_decode for callers that cannot hand over a scratch buffer.  No counterpart in the
 * reference.  Meant for hosts that own no device allocator of their own: a plugin living inside a
 * serving process whose memory pool is private to that process, or a latency-critical loop where
 * cudaMalloc/cudaFree are ruled out once the service is up (they stall the device and can fail
 * when memory is fragmented).  Inputs and outputs are still the caller's; only the per-split
 * partial results go to an array built into the library (nf4_b200_attn_decode_static_max_bytes()
 * = 4,259,840 bytes, enough for B=16, Hq=64, nsplit=8; each GPU that loads the library holds it
 * until exit).  A shape that needs more is refused with NF4_ERR_LIMIT.  The function performs no
 * device allocation or free.
 *   - The first call on a device looks up the array's device address (with that device current)
 *     and remembers it; make that first call before starting any stream capture.
 *   - All calls share the one array and it keeps whatever the last call left there.  Nothing has
 *     to be cleared: each call writes every slot before reading it.  Two calls that are in flight
 *     on the GPU at the same time (different streams, or different threads) overwrite each
 *     other's partial results -- serialise them.
 */
int nf4_b200_attn_decode_static(const void* q, const void* k_cache, const void* v_cache, const int* positions,
                                void* out, int64_t B, int Hq, int Hkv, int Dh, int64_t S_max, int nsplit, void* stream);
int64_t nf4_b200_attn_decode_static_max_bytes(void);
/* gate_up [rows, 2F] -> h [rows, F]: interleaved == 0: h[r,i] = silu(gate_up[r,i]) * gate_up[r,F+i];
 * interleaved != 0: h[r,i] = silu(gate_up[r,2i]) * gate_up[r,2i+1] */
int nf4_b200_silu_mul(const void* gate_up, void* h, int64_t rows, int64_t F, int interleaved, void* stream);
/* y = a + b (numel even) */
int nf4_b200_add(const void* a, const void* b, void* y, int64_t numel, void* stream);
/* y[r,:] = table[ids[r],:] */
int nf4_b200_embed(const int64_t* ids, const void* table, void* y, int64_t rows, int64_t D, int64_t vocab, void* stream);
/* ids[r] = argmax_v logits[r,v], the first maximum wins */
int nf4_b200_argmax(const void* logits, int64_t* ids, int64_t rows, int64_t V, void* stream);

/*
 * One-shot all-reduce (sum) of a small bf16 tile over peer memory, for the partial outputs of the row-parallel
 * projections of a tensor-parallel decode step.  In the reference this exchange is an NCCL all-reduce issued by
 * the torch executor (thunder/executors/torchex.py:2058-2078) after a row-parallel linear
 * (thunder/distributed/tensor_parallel/row_wise.py:53-80); here every rank stores its tile into a buffer of every
 * other rank and adds the `world` tiles it received, in rank order, so all ranks get identical bits:
 *     y = sum_r partial_r (+ residual)          fp32 sums, one rounding to bf16; y may alias residual or partial
 *   host_buffer_ptrs  HOST array of `world` device addresses: the buffer of rank r as mapped into THIS process
 *                     (entry `rank` is the caller's own).  Every buffer has buffer_bytes >=
 *                     nf4_b200_tp_allreduce_buffer_bytes(max numel) bytes, is zero-filled once before its first use
 *                     and is used by nothing else.  All ranks must issue the same sequence of calls (same numel).
 *   numel             elements of the tile, a multiple of 8; world <= 8.
 *   flags             bit 0: programmatic dependent launch (see nf4_b200_gemv_decode): the call may start while the
 *                     kernel that produces `partial` is finishing, and lets the next kernel of the stream start early.
 * The kernel writes to peers with plain stores and reads only its own memory; its waits on the peers' flags are
 * bounded (0.5 s): a wait that runs out records code 10 in nf4_b200_device_error ([1] block, [2] the rank that did
 * not arrive) and the call completes with incomplete sums instead of hanging.  Calls on one buffer set must not
 * overlap on the GPU (one stream).  nf4_b200_tp_allreduce_emulated runs ALL ranks of one exchange on the current
 * device in a single cooperative launch (arrays indexed by rank): for testing the protocol on one GPU.
 */
int64_t nf4_b200_tp_allreduce_buffer_bytes(int64_t max_numel);
int nf4_b200_tp_allreduce(const void* partial, const void* residual, void* y, int64_t numel, const uint64_t* host_buffer_ptrs,
                          int64_t buffer_bytes, int rank, int world, int flags, void* stream);
int nf4_b200_tp_allreduce_emulated(const uint64_t* host_partial_ptrs, const uint64_t* host_residual_ptrs,
                                   const uint64_t* host_y_ptrs, int64_t numel, const uint64_t* host_buffer_ptrs,
                                   int64_t buffer_bytes, int world, void* stream);

/*
 * Status word of the kernels that wait on in-kernel barriers (the staged GEMV).  Copies 4 words to
 * host memory: [0] first error code (0 = none; GEMV: 1/2/3 = a bounded wait on a full/empty/activation
 * barrier ran out, 4 = unexpected shared-memory window; GEMM: 5/6/7/8 = a bounded wait on the
 * full/empty/weights-ready/accumulator barrier ran out; attention / rotary kernels: 9 = a position outside
 * [0, S_max), then [1] is the batch row and [2] the position; all-reduce: 10 = a peer's flag did not arrive, [2] is
 * that peer's rank), [1] block index, [2] pipeline stage,
 * [3] number of waits that ran out.  SYNCHRONISES the device; for tests and diagnosis only.  No
 * counterpart in the reference.
 */
int nf4_b200_device_error(unsigned int* host_out4);
/* Sets the status words of the current device back to "no error" (synchronises).  The words are sticky: the
 * first error stays until this call, so that a caller who polls rarely still sees it. */
int nf4_b200_device_error_clear(void);

#ifdef __cplusplus
}
#endif
#endif /* NF4_B200_H */
