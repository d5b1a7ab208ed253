/*
 * awq_b200.h -- C ABI of libawq_b200.so: AWQ W4A16 linear and fused-MoE kernels for
 * NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (cudaStream_t passed
 * as void*); no framework types cross this boundary.  The caller owns every buffer,
 * including scratch; the library allocates nothing, keeps no pointer after the call returns
 * and never synchronises the stream.  All work is enqueued on `stream`.
 *
 * Most kernels are launched with CUDA's programmatic-stream-serialisation attribute: a kernel of
 * this library that follows another one on the stream starts early, prefetches weights (which
 * no kernel writes) and waits for the earlier kernel to complete before it reads activations or
 * writes anything.  Stream order as the caller sees it is unchanged; the weights passed to a
 * call must not be written by work still in flight on the same stream.  AWQ_B200_NO_PDL in the
 * environment (read once) makes every launch a plain one.
 *
 * Return value: AWQ_B200_OK (0) or a negative AWQ_B200_ERR_* code.  Arguments are validated on
 * the host before anything is launched; a kernel never traps.
 *
 * Tensor conventions (identical to vLLM's AWQ checkpoints; paths below are inside the vllm
 * package, version 0.22.0, which is the arithmetic the cloudrift-ai/server-benchmark harness
 * measures through the `vllm/vllm-openai` image: utils/generate_compose.py:65-100,
 * benchmarks/3_vllm_benchmark.sh:151-162):
 *   qweight int32 [K, N/8]      8 int4 per word along N, nibble p (LSB first) = column
 *                               [0,2,4,6,1,3,5,7][p] of the word's 8 columns
 *   qzeros  int32 [K/G, N/8]    same packing
 *   scales  fp16  [K/G, N]
 *   W[k][n] = (q[k][n] - z[k/G][n]) * s[k/G][n]
 *   (model_executor/layers/quantization/awq.py:182-255, awq_triton.py:54-101)
 */
#ifndef AWQ_B200_H_
#define AWQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AWQ_B200_OK 0
#define AWQ_B200_ERR_NULL (-1)      /* a required pointer is NULL */
#define AWQ_B200_ERR_SHAPE (-2)     /* a size is non-positive or violates a divisibility rule */
#define AWQ_B200_ERR_ALIGN (-3)     /* a pointer is not 16-byte aligned */
#define AWQ_B200_ERR_GROUP (-4)     /* unsupported quantisation group size */
#define AWQ_B200_ERR_WORKSPACE (-5) /* scratch buffer missing or too small */
#define AWQ_B200_ERR_LAUNCH (-6)    /* the CUDA runtime refused a launch */
#define AWQ_B200_ERR_DEVICE (-7)    /* current device is not compute capability 10.x */
#define AWQ_B200_ERR_DRIVER (-8)    /* a driver entry point (tensor-map encode) is unavailable */
#define AWQ_B200_ERR_LIMIT (-9)     /* a size exceeds a fixed built-in capacity */
#define AWQ_B200_ERR_SYMBOL (-10)   /* the built-in scratch array could not be bound on this GPU */

/* Human-readable text for a return code.  Never NULL. */
const char* awq_b200_strerror(int code);

/* Library version, "major.minor". */
const char* awq_b200_version(void);

/*
 * W fp16 [K, N] = (q - z) * s, the product rounded once to fp16.
 * Replaces torch.ops._C.awq_dequantize(qweight, scales, zeros, split_k_iters, thx, thy)
 * (vllm/_custom_ops.py:542-556; called from quantization/awq.py:280).
 * Requires N % 8 == 0, K % group == 0, group % 8 == 0.
 */
int awq_b200_dequantize(const void* qweight, const void* scales, const void* qzeros, void* out,
                        int K, int N, int group, void* stream);

/*
 * y fp16 [M, N] = x fp16 [M, K] @ W, fp32 accumulation, optional fp16 bias [N] added before
 * the final rounding (bias may be NULL).
 * Replaces torch.ops._C.awq_gemm(input, qweight, scales, qzeros, split_k_iters)
 * (vllm/_custom_ops.py:576-587; called from quantization/awq.py:283) and the
 * awq_dequantize + torch.matmul pair used for >= 256 tokens (awq.py:276-281): one entry
 * point serves every M, picking a weight-streaming kernel or one of the tcgen05 kernels by M.
 * `kernel` selects the implementation: AWQ_B200_KERNEL_AUTO or one of the explicit ids (a
 * request the shape does not permit returns AWQ_B200_ERR_SHAPE).
 * Scratch: awq_b200_gemm_workspace_bytes(M, N, K, group, kernel) bytes, 256-byte aligned; may
 * be NULL when that size is 0.
 */
#define AWQ_B200_KERNEL_AUTO 0
#define AWQ_B200_KERNEL_GENERIC 1  /* CUDA-core reference kernel, any legal shape */
#define AWQ_B200_KERNEL_STREAM 2   /* small-M weight-streaming kernel (mma.sync, cluster split-K) */
#define AWQ_B200_KERNEL_TCGEN05 3  /* large-M tcgen05/TMEM kernel with in-smem dequantisation */
#define AWQ_B200_KERNEL_STREAM_EXACT 4 /* small-M kernel with the magic-number conversion */
#define AWQ_B200_KERNEL_TS 5       /* M <= 16: registers -> TMEM weights, tcgen05.mma (A in TMEM) */
#define AWQ_B200_KERNEL_TS_EXACT 6 /* the same with the magic-number conversion */
#define AWQ_B200_KERNEL_WT 7       /* any M: dequantised weights registers -> TMEM (A operand), x via TMA as B */
#define AWQ_B200_KERNEL_STREAM_RP 8 /* M <= 8 streaming kernel; `qweight` is the output of awq_b200_repack_qweight */
#define AWQ_B200_KERNEL_Q8 9 /* M <= 32: `qweight` is the output of awq_b200_repack_kmajor; nibbles widened by tcgen05.cp, int8 MMAs */

size_t awq_b200_gemm_workspace_bytes(int M, int N, int K, int group, int kernel);

/*
 * Optional load-time repack of qweight for the decode kernel (AWQ_B200_KERNEL_STREAM_RP):
 * out int32 [K/4, N/8, 4] holds, for every quad of rows and packed word column, the four
 * row-pair registers the in-kernel unpack otherwise builds with byte permutes -- a pure
 * permutation of the bits of qweight, same size.  K % 4 == 0.  The AWQ layout stays the layout of
 * every other kernel, so a caller that wants the faster decode kernel keeps both copies.
 * Counterpart in the reference stack: the load-time repack of the Marlin path
 * (quantization/awq_marlin.py:491-499), which this replaces for M <= 8; scales and qzeros are
 * used as they are.
 */
int awq_b200_repack_qweight(const void* qweight, void* out, int K, int N, void* stream);

/*
 * Load-time repack of qweight for AWQ_B200_KERNEL_Q8: the same nibbles, running along K instead of
 * along N, in tiles of 256 output columns x 128 k (one quantisation group) = 16 KB, tiles ordered
 * column slab outermost, group inside; row r of a tile is column 256 * slab + r, byte b of the row
 * holds k = 2 b (low nibble) and 2 b + 1 of the group.  Columns past N in the last slab are zero.
 * out: awq_b200_repack_kmajor_bytes(K, N) bytes, 32-byte aligned (0 = shape not supported).
 * Requires K % 128 == 0, N % 8 == 0; scales and qzeros are used as they are.
 * Counterpart in the reference stack: the load-time Marlin repack
 * (quantization/awq_marlin.py:491-499, awq_marlin.py:90-165), whose decode kernel this replaces.
 *
 * With that copy, awq_b200_gemm(kernel = AWQ_B200_KERNEL_Q8) never touches a weight from a
 * thread: TMA lays the packed nibbles into shared memory, tcgen05.cp widens them to bytes on the
 * way into tensor memory, tcgen05.mma.kind::i8 multiplies them with the activations rewritten
 * as 24-bit fixed point per token (three signed byte digits; a first small kernel of the call
 * does that), and only the per-group scale / zero fold runs on the CUDA cores.  M <= 32, group 128,
 * K <= 32768.  Its scratch (awq_b200_gemm_workspace_bytes with this kernel id) holds the digits and
 * the partial tiles CTAs hand to each other; calls that may overlap on the GPU need separate
 * scratch buffers.
 */
size_t awq_b200_repack_kmajor_bytes(int K, int N);

int awq_b200_repack_kmajor(const void* qweight, void* out, int K, int N, void* stream);

/*
 * Load-time conversion of stacked expert weights from the byte layout of vLLM's MoE WNA16 method
 * to the AWQ checkpoint layout the expert entry points below take.  In: w uint8 [E, N, K/2]
 * (k = 2j in the low nibble of byte j), scales fp16 [E, N, K/group], zeros uint8 [E, N/2, K/group]
 * (n = 2i in the low nibble of row i) -- the parameters MoeWNA16Method.create_weights declares
 * (quantization/moe_wna16.py:252-324).  Out: qweight int32 [E, K, N/8] and qzeros int32
 * [E, K/group, N/8] in AWQ nibble order, scales fp16 [E, K/group, N].  Bit-exact inverse of the
 * converter in that method's weight loader (moe_wna16.py:389-425).  N % 8 == 0, K % group == 0.
 */
int awq_b200_wna16_to_awq(const void* w, const void* scales, const void* zeros, void* qweight,
                          void* scales_out, void* qzeros, int E, int N, int K, int group,
                          void* stream);

int awq_b200_gemm(const void* x, const void* qweight, const void* scales, const void* qzeros,
                  const void* bias, void* out, int M, int N, int K, int group, int kernel,
                  void* workspace, size_t workspace_bytes, void* stream);

/*
 * Health word of the tcgen05 kernel on the current device.  Its mbarrier waits are bounded;
 * a wait that ran out records which one (1 producer, 2-3 MMA issuer, 4 dequantisation,
 * 5 epilogue; 11-15 the M <= 16 kernel) and the kernel tears down instead of hanging.  0 = no wait ever ran out.
 * Synchronises the device (a plain device-to-host copy).  No counterpart in the reference.
 */
int awq_b200_device_status(int* status);

/*
 * The same, and the word is put back to 0 afterwards.  The word is sticky: it keeps the first
 * wait that ran out (31-35: the AWQ_B200_KERNEL_Q8 kernel; 35 = a CTA waited in vain for a
 * partial tile of another CTA) until it is cleared here, and a call during which a wait ran out
 * still returns AWQ_B200_OK with an incomplete output.  No counterpart in the reference.
 */
int awq_b200_device_status_clear(int* status);

/*
 * Number of polls after which a CTA of the AWQ_B200_KERNEL_Q8 kernel stops waiting for another
 * CTA's partial tile (0 restores the default, 2^20), and after which awq_b200_allreduce stops
 * waiting for a peer (default 2^22).  Process-wide; meant for tests that check the
 * give-up path with a tiny limit.  No counterpart in the reference.
 */
void awq_b200_set_wait_limit(unsigned int polls);

/*
 * One-shot all-reduce (sum) of fp16 partial outputs over peer memory, for the row-parallel linears
 * of a tensor-parallel model: replaces the all-reduce behind RowParallelLinear.forward
 * (vllm/model_executor/layers/linear.py:1556-1559; vLLM's own small-message path is
 * distributed/device_communicators/custom_all_reduce.py:232-245).
 *
 * Every rank owns one region of device memory that all `world` ranks (one process per GPU, one
 * node) have mapped; regions[r] is rank r's region as mapped in THIS process (regions[rank] is
 * the local one).  A region starts with AWQ_B200_AR_FLAG_BYTES of flags, zero when the first call
 * is made; the partial of this call lies at `data_offset` (>= AWQ_B200_AR_FLAG_BYTES, a multiple
 * of 16, the same on all ranks) and is `bytes` long (a multiple of 16).  All ranks make the same
 * sequence of calls.  The kernel tells its peers that the partial is complete, waits for theirs,
 * adds the `world` partials in rank order in fp32 and writes fp16 to `out` (local memory).
 * `state`: 8 bytes of local device memory, zero before the first call, private to this sequence
 * of calls (it numbers the calls on the device, so a CUDA graph that holds the call can be
 * replayed).  flags: bit 0 = also wait, before returning, until every peer has finished reading
 * (needed when the next call uses the same data_offset; a caller that alternates between two
 * offsets does not need it: a rank cannot start call i+2 before every peer has left call i);
 * bit 1 = programmatic dependent launch after the kernel that writes the partial (measured 1.4 us
 * slower per call than a plain launch behind the decode GEMMs: off in the Python host).
 * Peer memory is read with plain loads; nothing is bound to a multicast object.  Waits are
 * bounded (awq_b200_set_wait_limit); one that runs out leaves 70 + peer (start) or 80 + peer
 * (end) in the status word, `out` incomplete, and the call numbering of the ranks out of step.
 */
#define AWQ_B200_AR_MAX_RANKS 8
#define AWQ_B200_AR_MAX_BLOCKS 32
#define AWQ_B200_AR_FLAG_BYTES 4096
int awq_b200_allreduce(const void* const* regions, int rank, int world, size_t data_offset,
                       void* out, size_t bytes, void* state, int flags, void* stream);

/*
 * Set-up of the regions awq_b200_allreduce works on, for one process per GPU on one node.
 * create: cudaMalloc of `bytes` (>= AWQ_B200_AR_FLAG_BYTES) on the current device, zeroed, and its
 *         CUDA IPC handle (AWQ_B200_IPC_HANDLE_BYTES bytes) for the other ranks.
 * open:   maps another rank's region from its handle into the CURRENT device's context
 *         (cudaIpcOpenMemHandle with lazy peer access: this process's kernels may then dereference
 *         it).  A handle cannot be opened by the process that created it.
 * close / destroy undo open / create.  The host moves the handles between processes itself (the
 * Python host uses torch.distributed.all_gather_object).  vLLM's counterpart:
 * distributed/device_communicators/custom_all_reduce.py:150-230 (buffer creation and handle exchange).
 */
#define AWQ_B200_IPC_HANDLE_BYTES 64
int awq_b200_peer_region_create(size_t bytes, void** region, void* handle);
int awq_b200_peer_region_open(const void* handle, void** region);
int awq_b200_peer_region_close(void* region);
int awq_b200_peer_region_destroy(void* region);

/*
 * Runs the give-up path of the bounded waits once: a one-warp kernel waits, with a limit of
 * `polls`, on an mbarrier nobody arrives on and then on a flag nobody sets.  Both waits run out,
 * the kernel returns normally, and awq_b200_device_status_clear then reports 90 (the first of
 * the two).  The context stays usable.  No counterpart in the reference.
 */
int awq_b200_selftest_wait(unsigned int polls, void* stream);

/*
 * Router: softmax over E experts, top-k (ties: lower expert id first), optional
 * renormalisation of the k weights.  gating is fp32 (gating_dtype 0) or fp16 (1), [T, E].
 * Outputs: topk_weights fp32 [T, k], topk_ids int32 [T, k], token_expert_indices int32 [T, k]
 * (= slot * T + token; may be NULL).
 * Replaces torch.ops._moe_C.topk_softmax (vllm/_custom_ops.py:2370-2385;
 * fused_moe/router/fused_topk_router.py:17-33).  Requires E <= 1024, k <= 32, k <= E.
 */
int awq_b200_topk_softmax(const void* gating, int gating_dtype, int T, int E, int topk,
                          int renormalize, float* topk_weights, int32_t* topk_ids,
                          int32_t* token_expert_indices, void* stream);

/*
 * Token -> expert permutation (stable counting sort).  sorted_ids receives the flat
 * (token * topk + slot) indices grouped by expert in ascending flat index, each expert's run
 * padded to a multiple of `block` with the sentinel T*topk; every remaining entry up to
 * `sorted_capacity` is the sentinel too.  expert_ids[b] is the expert of block b (-1 past the
 * used blocks), num_post_pad[0] the padded total.  expert_map (may be NULL) maps global to
 * local expert ids, -1 = not on this rank (those entries are dropped).
 * sorted_capacity must be >= awq_b200_moe_sorted_capacity(T * topk, E, block);
 * expert_ids holds ceil(sorted_capacity / block) entries.
 * Replaces torch.ops._moe_C.moe_align_block_size (vllm/_custom_ops.py:2247-2264;
 * fused_moe/moe_align_block_size.py:11-103).  Requires E <= 1024, T * topk <= 2^24.
 */
int64_t awq_b200_moe_sorted_capacity(int64_t numel, int E, int block);

int awq_b200_moe_align_block_size(const int32_t* topk_ids, int T, int topk, int E, int block,
                                  const int32_t* expert_map, int32_t* sorted_ids,
                                  int64_t sorted_capacity, int32_t* expert_ids,
                                  int32_t* num_post_pad, void* stream);

/*
 * AWQ fused-MoE experts: for every (token, slot) gate_up GEMM -> silu(gate) * up -> down GEMM
 * -> times routed weight -> sum over slots into out fp16 [T, H].
 *   w13_q int32 [E, H, 2I/8], w13_s fp16 [E, H/G, 2I], w13_z int32 [E, H/G, 2I/8]
 *   w2_q  int32 [E, I, H/8],  w2_s  fp16 [E, I/G, H],  w2_z  int32 [E, I/G, H/8]
 * (parameter layout: quantization/awq_marlin.py:549-623).  sorted_ids / expert_ids /
 * num_post_pad are the outputs of awq_b200_moe_align_block_size with block =
 * awq_b200_moe_block_size(T, topk, E, H, I, group): 8 or 16 (weight-streaming kernels; 8 while an
 * expert sees at most eight rows on average) for decode-size batches, 128 (tcgen05 grouped GEMMs)
 * once an expert sees 36 rows or more on average.
 * Replaces fused_experts / fused_experts_impl (fused_moe/fused_moe.py:1587-1631,1664-1869)
 * and the Marlin expert path (fused_moe/experts/marlin_moe.py:225-262).
 * E is the number of stacked (local) experts.  `expert_parallel` is a set of flags: bit 0 says
 * sorted_ids was built with an expert_map, i.e. some (token, slot) pairs have no expert here and
 * contribute zero; bit 1 says w13_q and w2_q are decode-layout copies (awq_b200_repack_qweight
 * over all E * H, respectively E * I, stacked rows), which only the weight-streaming kernels
 * read: block 8 or 16 and group 128, anything else returns AWQ_B200_ERR_SHAPE; bit 2 selects the
 * direct mode for a handful of pairs (T * topk <= AWQ_B200_MOE_DIRECT_MAX_PAIRS, block 8, no
 * expert_map): no permutation is needed - expert_ids is the routed-id table topk_ids [T * topk]
 * itself, sorted_ids and num_post_pad are ignored (may be NULL), sorted_capacity must be
 * T * topk * 8 (one 8-row block per pair) - which takes awq_b200_moe_align_block_size out of the
 * chain for the decode of one or two tokens; the down GEMM then also adds a token's slots itself
 * (the cluster that finishes the token's last pair for a column slab, counted in 4 KB of
 * counters at the end of the scratch layout that the first GEMM of the call clears), so the chain
 * is two launches.  Every routed id must be a valid expert index in this mode, and the scratch
 * need (one 8-row block per pair) exceeds the bound of awq_b200_moe_workspace_bytes once
 * T * topk * 8 > awq_b200_moe_sorted_capacity(T * topk, E, 16): size the buffer for the layout.
 * Scratch, 256-byte aligned: the activation and per-pair buffers are laid out for
 * round_up(sorted_capacity, block) rows, so the size needed follows the sorted_capacity passed
 * here.  awq_b200_moe_workspace_bytes(T, topk, E', H, I) bounds it when sorted_capacity is
 * awq_b200_moe_sorted_capacity(T * topk, E', block) - with E' the expert count the permutation
 * was built for (the global count under expert parallelism, else E).  A buffer smaller than the
 * layout returns AWQ_B200_ERR_WORKSPACE before anything is launched.
 * Requires H % 128 == 0, I % 128 == 0, group in {32, 64, 128}.
 */
#define AWQ_B200_MOE_DIRECT_MAX_PAIRS 64
int awq_b200_moe_block_size(int T, int topk, int E, int H, int I, int group);

size_t awq_b200_moe_workspace_bytes(int T, int topk, int E, int H, int I);

int awq_b200_moe_experts(const void* x, const void* w13_q, const void* w13_s, const void* w13_z,
                         const void* w2_q, const void* w2_s, const void* w2_z,
                         const float* topk_weights, const int32_t* sorted_ids,
                         const int32_t* expert_ids, const int32_t* num_post_pad, void* out,
                         int T, int topk, int E, int H, int I, int group, int block,
                         int expert_parallel, int64_t sorted_capacity, void* workspace,
                         size_t workspace_bytes, void* stream);

/*
 * awq_b200_moe_experts with no scratch argument, for hosts that cannot obtain device memory at
 * call time.  (No counterpart in the reference: its Python callers always allocate through
 * torch.)  Examples: a serving engine that has already handed every free byte of HBM to its
 * KV-cache pool, so a late cudaMalloc would fail; a C or FFI host that has no device allocator
 * of its own and must not call the CUDA allocation routines from its request loop.
 *
 * The activation and per-pair buffers live in one array inside the library, in device memory,
 * awq_b200_moe_static_scratch_bytes() = 16 MiB per GPU.  The CUDA runtime binds it on a GPU at
 * the first use of the library's MoE code there (module loading is lazy) and keeps it for as long
 * as the process runs.  Inputs and the output are still the caller's.
 * Arguments are those of awq_b200_moe_experts without workspace / workspace_bytes.
 *
 *  - A problem whose scratch need exceeds the 16 MiB is refused with AWQ_B200_ERR_LIMIT before
 *    anything is launched (Qwen3-30B-A3B shapes fit up to about 300 tokens); the need is that of
 *    awq_b200_moe_experts and follows sorted_capacity in the same way.  Use
 *    awq_b200_moe_experts with your own buffer for larger problems.
 *  - The call never allocates or frees device memory.  The first call on each GPU looks up the
 *    array's device address (one cudaGetSymbolAddress, cached per GPU under a mutex), which is
 *    also when the array gets bound: that first call is mandatory during start-up, while
 *    device memory is still available and before any stream capture.  If the binding fails the
 *    call returns AWQ_B200_ERR_SYMBOL.
 *  - All calls on one GPU share the one array and it keeps the previous call's contents.  What
 *    has to start from zero is cleared by the call itself.  Two calls that overlap on the GPU
 *    (different streams, or a graph replay racing a direct call) corrupt each other: keep calls
 *    on one GPU ordered.
 */
size_t awq_b200_moe_static_scratch_bytes(void);

int awq_b200_moe_experts_static(const void* x, const void* w13_q, const void* w13_s,
                                const void* w13_z, const void* w2_q, const void* w2_s,
                                const void* w2_z, const float* topk_weights,
                                const int32_t* sorted_ids, const int32_t* expert_ids,
                                const int32_t* num_post_pad, void* out, int T, int topk, int E,
                                int H, int I, int group, int block, int expert_parallel,
                                int64_t sorted_capacity, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AWQ_B200_H_ */
