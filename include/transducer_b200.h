/*
 * transducer_b200 -- C ABI of the sm_100a RNN-T loss / Viterbi library.
 *
 * Drop-in boundary for the CUDA path of awni/transducer.  The first three entry
 * points take exactly the arguments of that project's transducer.h (minus the
 * `useCuda` flag: this library has no CPU backend); the remaining ones replace the
 * arithmetic its Python wrapper performs with torch ops around those calls.
 *
 * Conventions (identical to the reference, transducer/transducer_cpu.cpp:242-256):
 *   emissions    float [B, maxT, V]      unnormalised scores per frame
 *   predictions  float [B, maxU, V]      maxU = longest label sequence + 1
 *   labels       int   [B, maxU-1]
 *   inputLengths int   [B]               T_b  <= maxT
 *   labelLengths int   [B]               U_b = labelLengths[b] + 1 <= maxU
 *   lattices (logNorms, alphas, lngrads) float [B, maxT, maxU]
 * The output distribution at node (t,u) is log_softmax(E[b,t,:] + P[b,u,:]).
 *
 * All pointers are DEVICE pointers on the current device unless stated otherwise.
 * Calls are asynchronous on the stream chosen with tb200_set_stream (default: the
 * legacy default stream, as the reference launches on, transducer_cuda.cu:295).
 * Every function returns 0 on success, a TB200_ERR_* code otherwise; the message is
 * available from tb200_last_error() on the calling thread.
 */
#ifndef TRANSDUCER_B200_H_
#define TRANSDUCER_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TB200_OK 0
#define TB200_ERR_INVALID_ARGUMENT 1
#define TB200_ERR_CUDA 2
#define TB200_ERR_WORKSPACE 3
#define TB200_ERR_UNSUPPORTED 4
#define TB200_ERR_DEVICE_STATUS 5

/* Library version (major*10000 + minor*100 + patch). */
int tb200_version(void);

/* Message of the last failing call on this thread ("" if none). */
const char* tb200_last_error(void);

/* Stream (a cudaStream_t) used by subsequent calls from this thread.  NULL selects
 * the legacy default stream, which is what the reference's launches use
 * (transducer/transducer_cuda.cu:295,333,372).  No counterpart in the reference. */
int tb200_set_stream(void* stream);
void* tb200_get_stream(void);

/* Tuning / test switches.  Keys:
 *   "lognorm_path"  0 auto, 1 exact SIMT logsumexp, 2 tensor-core factored GEMM
 *   "grads_path"    0 auto, 1 SIMT, 2 tensor-core
 *   "grad_passes"   operand precision of the tensor-core gradient kernel.  The lattice
 *                   weights are always rounded once to TF32.  1: exp(E), exp(P) rounded
 *                   once too; 2 (default): exp(E) split hi+lo (exact products for
 *                   pgrads); 3: exp(P) split as well (smaller tiles, slower)
 *   "fused_gather"  1 (default): the tensor-core log-normaliser also hands out E[t,label_u] and
 *                   E[t,blank] from the rows it streams; 0: a separate gather pass fetches them
 *   "maxplus_path"  label-arc scores of the Viterbi pass (tb200_label_arc_scores): 0 auto,
 *                   1 the full loop over the alphabet, 2 candidate lists with an exact bound
 * Unknown keys return TB200_ERR_INVALID_ARGUMENT.  No counterpart in the reference. */
int tb200_set_option(const char* key, int value);
int tb200_get_option(const char* key, int* value);

/* Launch accounting.  tb200_launch_count: kernels launched by this library since
 * load.  With profiling enabled every launch is bracketed by CUDA events on its
 * stream; tb200_profile_report synchronises them and writes one
 * "kernel_name launches total_ms" line per kernel into buf (truncated to bufBytes,
 * NUL-terminated) and returns the untruncated length.  No counterpart in the
 * reference (it has wall-clock helpers only, transducer/benchmark_cuda.cu:59-74). */
long long tb200_launch_count(void);
int tb200_profile_enable(int on);
int tb200_profile_reset(void);
size_t tb200_profile_report(char* buf, size_t bufBytes);

/* Device-side failure detection.  Every wait inside the kernels (on a TMA / bulk copy, an MMA
 * completion, a pipeline stage) is bounded; a wait that runs out makes its kernel record a code
 * in a per-device status word, poison its outputs (NaN costs, log-normalisers and gradients,
 * labels of -1) and return normally, so the CUDA context stays usable.  tb200_check_status
 * SYNCHRONISES the calling thread's stream, reads the word of the current device, clears it,
 * and returns TB200_ERR_DEVICE_STATUS (message with the code in tb200_last_error()) if any
 * kernel of this library on this device gave up since the last check, else 0.  The word is
 * shared by all streams and threads using the device.  tb200_status_name: text for a code.
 * tb200_selftest_wait_timeout enqueues one tiny kernel that waits, for at most the given
 * number of microseconds, on a barrier that nothing ever completes: the next
 * tb200_check_status must then report code 5 -- the supported way of exercising this path
 * (it neither faults nor hangs the GPU).  The first call on a device looks up the word's
 * address (make it outside stream capture).
 * The reference has no device-side waits; its counterpart on the host is
 * cudaCheck -> std::runtime_error (transducer/transducer_cuda.cu:271-278). */
int tb200_check_status(void);
const char* tb200_status_name(int code);
int tb200_selftest_wait_timeout(unsigned limitMicroseconds);

/* ---- the reference's three entry points ------------------------------------ */

/* transducer/transducer.h:3-17 (`forward`, useCuda=true): alpha recursion.
 * Writes costs[B] (+inf where T_b==0) and the valid region of alphas. */
int tb200_forward(const float* emissions, const float* predictions, float* costs,
                  float* alphas, const float* logNorms, const int* labels,
                  const int* inputLengths, const int* labelLengths, int batchSize,
                  int maxInputLength, int maxLabelLength, int alphabetSize, int blank);

/* transducer/transducer.h:19-35 (`backward`): zero-fills egrads/pgrads/lngrads over
 * their full padded extent, then writes the node occupancies to lngrads and
 * subtracts the sparse blank/label terms from egrads/pgrads. */
int tb200_backward(const float* emissions, const float* predictions, float* egrads,
                   float* pgrads, float* lngrads, const float* alphas,
                   const float* logNorms, const int* labels, const int* inputLengths,
                   const int* labelLengths, int batchSize, int maxInputLength,
                   int maxLabelLength, int alphabetSize, int blank);

/* transducer/transducer.h:37-49 (`viterbi`): best alignment given the label
 * lengths; writes the first labelLengths[b] entries of labels[b,:].  Like the
 * reference (transducer_cuda.cu:364-369) it takes its temporaries from the
 * stream-ordered allocator. */
int tb200_viterbi(const float* emissions, const float* predictions,
                  const float* logNorms, int* labels, const int* inputLengths,
                  const int* labelLengths, int batchSize, int maxInputLength,
                  int maxLabelLength, int alphabetSize, int blank);

/* tb200_viterbi for callers that cannot allocate device memory.  It has no counterpart in
 * the reference (whose viterbi always calls cudaMallocAsync, transducer_cuda.cu:364-369).
 *
 * Who needs it: a host process whose device memory is entirely claimed by another
 * allocator (a framework's caching allocator, a server's fixed arena), so that the
 * driver's stream-ordered pool has nothing left to give; a device or virtual GPU without
 * memory-pool support, where cudaMallocAsync does not exist; a decoding loop that cannot
 * afford an allocation's occasional pool growth or synchronisation.
 *
 * Same arguments and result as tb200_viterbi.  The temporaries live in a fixed array inside
 * the library (about 17 MiB, resident on every GPU that loads the library until the process
 * ends), so the lattice is limited to tb200_viterbi_static_max_nodes() =
 * 4 Mi nodes of batchSize*maxInputLength*maxLabelLength (and 160 Ki back-pointer words,
 * batchSize*maxLabelLength*ceil(maxInputLength/32)); larger calls return
 * TB200_ERR_WORKSPACE without touching anything.  The call itself requests no memory from
 * any allocator (no cudaMalloc / cudaMallocAsync / cudaFree, no library routine that would).
 * The first call on each device looks up the array's device address and caches it; with the
 * CUDA runtime's lazy module loading that first call is also when the driver brings this
 * library's kernels and the array itself onto the device.  So make the first call per device
 * at start-up -- with the device current, before another allocator claims the rest of the
 * card, and before any stream capture begins -- a call with batchSize = 0 will do.
 * All calls share the one array and it keeps whatever the last call left (nothing in it
 * needs to be zero on entry), so two calls whose GPU work may overlap -- different streams,
 * different host threads -- race with each other: serialise them. */
size_t tb200_viterbi_static_max_nodes(void);
int tb200_viterbi_static(const float* emissions, const float* predictions,
                         const float* logNorms, int* labels, const int* inputLengths,
                         const int* labelLengths, int batchSize, int maxInputLength,
                         int maxLabelLength, int alphabetSize, int blank);

/* ---- the arithmetic the reference does in torch ops ------------------------- */

/* transducer/torch_binding.py:35-40 and :162-167: logNorms[b,t,u] =
 * logsumexp_v(E[b,t,v] + P[b,u,v]) for every valid node (padding is not written).
 * Also returns the per-row shifts the factored gradient kernels reuse:
 * rowRef [B,maxT] (a per-frame reference value <= max_v E, not necessarily the
 * maximum) and maxP [B,maxU].  workspace: tb200_log_norms_workspace_bytes(). */
size_t tb200_log_norms_workspace_bytes(int batchSize, int maxInputLength,
                                       int maxLabelLength, int alphabetSize);
int tb200_log_norms(const float* emissions, const float* predictions, float* logNorms,
                    float* rowRef, float* maxP, const int* inputLengths,
                    const int* labelLengths, int batchSize, int maxInputLength,
                    int maxLabelLength, int alphabetSize, void* workspace,
                    size_t workspaceBytes);

/* transducer/torch_binding.py:25-58 (Transducer.forward): log-normalisers + alpha
 * recursion.  Writes costs[B]; if lossSum is not NULL it receives sum_b costs[b]
 * (added in index order by the last CTA to finish).  What the reference keeps for
 * its backward pass as autograd-saved tensors (alphas, log_norms, expEs, ...,
 * torch_binding.py:52-55) is kept here in `saved`, an opaque device buffer of
 * tb200_loss_saved_bytes() owned by the caller; exp(E) is not among it. */
size_t tb200_loss_saved_bytes(int batchSize, int maxInputLength, int maxLabelLength,
                              int alphabetSize);
size_t tb200_loss_forward_workspace_bytes(int batchSize, int maxInputLength,
                                          int maxLabelLength, int alphabetSize);
int tb200_loss_forward(const float* emissions, const float* predictions,
                       const int* labels, const int* inputLengths,
                       const int* labelLengths, float* costs, float* lossSum,
                       void* saved, size_t savedBytes, int batchSize,
                       int maxInputLength, int maxLabelLength, int alphabetSize,
                       int blank, void* workspace, size_t workspaceBytes);

/* transducer/torch_binding.py:60-90 (Transducer.backward): reverse sweep + dense
 * gradient contractions + deltas scaling, from the same inputs and the `saved`
 * buffer of the forward call.  Every element of egrads [B,maxT,V] and pgrads
 * [B,maxU,V] is written (zeros in the padding).  egrads may be the emissions buffer itself
 * and pgrads the predictions buffer (gradients in place: every tile is read before it is
 * written and nothing else in the call reads them) whenever the tensor-core gradient kernel
 * runs (alphabetSize % 4 == 0, maxLabelLength <= 128, 16-byte aligned buffers); otherwise
 * aliasing is refused with TB200_ERR_INVALID_ARGUMENT. */
size_t tb200_loss_backward_workspace_bytes(int batchSize, int maxInputLength,
                                           int maxLabelLength, int alphabetSize);
int tb200_loss_backward(const float* emissions, const float* predictions,
                        const int* labels, const int* inputLengths,
                        const int* labelLengths, const void* saved, size_t savedBytes,
                        const float* deltas, float* egrads, float* pgrads,
                        int batchSize, int maxInputLength, int maxLabelLength,
                        int alphabetSize, int blank, void* workspace,
                        size_t workspaceBytes);

/* The same two calls for bf16 storage: emissions, predictions and both gradients are bfloat16
 * in memory (2 bytes per element), which halves the bytes the path streams.  Every value is
 * converted exactly to fp32 on the way in, all arithmetic and everything in `saved` is the
 * fp32 path's, and the gradients are rounded to nearest on the way out: the results are those
 * of tb200_loss_forward / tb200_loss_backward on the up-converted inputs, the gradients rounded
 * once.  The reference takes fp32 only (transducer/torch_binding.py:195-197).  Needs
 * alphabetSize % 8 == 0, maxLabelLength <= 128, 16-byte aligned buffers, and the default
 * "grad_passes" = 2; otherwise TB200_ERR_INVALID_ARGUMENT.  Saved / workspace sizes are those
 * of the fp32 calls. */
int tb200_loss_forward_bf16(const void* emissions, const void* predictions,
                            const int* labels, const int* inputLengths,
                            const int* labelLengths, float* costs, float* lossSum,
                            void* saved, size_t savedBytes, int batchSize,
                            int maxInputLength, int maxLabelLength, int alphabetSize,
                            int blank, void* workspace, size_t workspaceBytes);
int tb200_loss_backward_bf16(const void* emissions, const void* predictions,
                             const int* labels, const int* inputLengths,
                             const int* labelLengths, const void* saved, size_t savedBytes,
                             const float* deltas, void* egrads, void* pgrads,
                             int batchSize, int maxInputLength, int maxLabelLength,
                             int alphabetSize, int blank, void* workspace,
                             size_t workspaceBytes);

/* transducer/transducer_cuda.cu:233-242, transducer_cpu.cpp:156-169 (the loop over the
 * alphabet inside the Viterbi sweep), for every lattice node at once:
 * best[b,t,u] = max over v != blank of emissions[b,t,v] + predictions[b,u,v], written for
 * t < inputLengths[b], u < labelLengths[b] (row-major [batchSize, maxInputLength,
 * maxLabelLength]; other entries untouched).  Alphabets of 1024 words and more are evaluated
 * from per-frame and per-position candidate lists with an exact bound (bit-identical to the
 * full loop; nodes the bound does not settle are evaluated in full);
 * tb200_set_option("maxplus_path", 1) forces the full loop, 2 the lists. */
size_t tb200_label_arc_scores_workspace_bytes(int batchSize, int maxInputLength,
                                              int maxLabelLength, int alphabetSize);
int tb200_label_arc_scores(const float* emissions, const float* predictions,
                           const int* inputLengths, const int* labelLengths, float* best,
                           int batchSize, int maxInputLength, int maxLabelLength,
                           int alphabetSize, int blank, void* workspace,
                           size_t workspaceBytes);

/* transducer/torch_binding.py:130-177 (TransducerLoss.viterbi): log-normalisers +
 * best path, all temporaries in the caller's workspace. */
size_t tb200_viterbi_decode_workspace_bytes(int batchSize, int maxInputLength,
                                            int maxLabelLength, int alphabetSize);
int tb200_viterbi_decode(const float* emissions, const float* predictions,
                         const int* inputLengths, const int* labelLengths, int* labels,
                         int batchSize, int maxInputLength, int maxLabelLength,
                         int alphabetSize, int blank, void* workspace,
                         size_t workspaceBytes);

/* The path's one collective without a collective library: the per-rank loss sums (4 bytes
 * each) exchanged by plain peer stores over NVLink, one launch of one warp per rank and step.
 * The reference is single-GPU (nothing to cite); the usual route is an all-reduce of the
 * lossSum that tb200_loss_forward wrote (NCCL), which this replaces.
 *
 * Every rank (one process per GPU) owns a slot buffer: tb200_peer_alloc (cudaMalloc'ed, zeroed,
 * tb200_peer_slots_bytes() bytes); tb200_peer_export writes its 64-byte CUDA IPC handle, which
 * the caller sends to the other ranks by any means; tb200_peer_import opens a peer's handle
 * (peer access is enabled on demand) and tb200_peer_close / tb200_peer_free undo the two.
 * tb200_loss_sum_exchange, called by every rank with the same seq = 1, 2, 3, ... (one per
 * step) and peerSlots[r] = rank r's buffer as seen from this process (its own for r == rank):
 * stores (seq, *lossSum) into every rank's buffer, waits until its own buffer holds all ranks'
 * values of this seq, and writes their sum, added in rank order (identical bits on every
 * rank), to *total.  Asynchronous on the current stream like every other call.  A peer whose
 * value does not arrive within timeoutUs microseconds (0: the library's 2 s limit) makes
 * *total NaN and is reported by tb200_check_status; the context stays usable.  world <= 32. */
size_t tb200_peer_slots_bytes(void);
int tb200_peer_alloc(void** slots);
int tb200_peer_free(void* slots);
int tb200_peer_export(const void* slots, void* handle64);
int tb200_peer_import(const void* handle64, void** slots);
int tb200_peer_close(void* slots);
int tb200_loss_sum_exchange(const float* lossSum, void* const* peerSlots, int rank, int world,
                            unsigned seq, float* total, unsigned timeoutUs);

#ifdef __cplusplus
}
#endif
#endif /* TRANSDUCER_B200_H_ */
