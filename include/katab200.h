/* C ABI of libkatab200.so: the B200 (sm_100a) implementation of the KataGo neural-net
 * forward pass that sits below the reference's backend interface
 * (cpp/neuralnet/nninterface.h:32-182).  The reference-side backend
 * (katago_b200/host/b200backend.cpp) and the Python harness (katago_b200/capi.py) both
 * bind exactly these entry points.
 *
 * Conventions: plain pointers and sizes only; every function returns 0 on success and a
 * non-zero code on failure, never throws; the message of the last failure on the calling
 * thread is available from kb_last_error().  A kb_handle is bound to one GPU and must be
 * used by one thread at a time (nninterface.h:19-21).  There is no CPU fallback: without
 * a CUDA device every compute entry point fails.
 */
#ifndef KATAB200_H_
#define KATAB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct kb_model kb_model;   /* parsed network, host memory, device independent */
typedef struct kb_handle kb_handle; /* one GPU replica: device weights, activations, stream */

enum { KB_PRECISION_FP32 = 0, KB_PRECISION_FP16 = 1, KB_PRECISION_BF16 = 2 };

/* Message of the last failure on the calling thread (never NULL). */
const char* kb_last_error(void);

/* Library version string. */
const char* kb_version(void);

/* Replaces NeuralNet::printDevices / device selection (nninterface.h:39, cudabackend.cpp:3333). */
int kb_device_count(int* count);
int kb_device_name(int device, char* buf, size_t buflen);

/* Replaces the construction of the backend's Model from a ModelDesc
 * (nninterface.h:43-46 loadModelFile/getModelDesc feed it; cudabackend.cpp:2852-2963).
 * `blob` is the record stream of include/kb_modelblob.h. */
int kb_model_create(const void* blob, size_t nbytes, kb_model** out);
void kb_model_destroy(kb_model* m);

/* info[0..8] = modelVersion, inC, inGlobalC, policyC, valueC, scoreValueC, ownershipC, trunkC, numBlocks */
int kb_model_info(const kb_model* m, int32_t info[9]);
/* Number of SGF metadata input channels (ModelDesc::numInputMetaChannels, desc.h; 0 for nets without the encoder). */
int kb_model_meta_channels(const kb_model* m, int32_t* channels);

/* Replaces NeuralNet::createComputeHandle / freeComputeHandle (nninterface.h:76-86):
 * binds the calling thread to `device` (-1 = current default), uploads the weights in the
 * chosen precision and allocates every activation buffer for batches up to maxBatch.
 * requireExactNNLen != 0 promises that every board is exactly nnXLen x nnYLen. */
int kb_handle_create(
  const kb_model* m, int device, int maxBatch, int nnXLen, int nnYLen, int precision, int requireExactNNLen,
  kb_handle** out);
void kb_handle_destroy(kb_handle* h);

/* Device-side weight cache.  The reference's CPU backend shares one Model between all compute handles of a net,
 * keyed by name and hash (eigenbackend.cpp:2364-2392), so that several server threads cost one copy of the weights;
 * here every read-only weight tensor is keyed by device and contents, reference counted, and freed with the last
 * handle that uses it: handles created from the same model on the same device hold one replica between them.
 * stats[0..3] = live entries, their bytes, uploads made, uploads avoided (since the process started, all devices). */
int kb_weight_cache_stats(int64_t stats[4]);

/* The tile plan of a tensor-core convolution kY x kX = k x k, inC -> outC (inC as the device sees it: padded to a multiple
 * of 64).  Replaces the OpenCL backend's start-up autotuner (cpp/neuralnet/opencltuner.cpp) by a committed table
 * (katago_b200/csrc/kb_tile_table.h).  Host-only.  plan[0..5] = channels per tile (N of the MMA), CTA pairs (0/1), epilogue
 * warps per TMEM lane quarter without / with a residual, multi-layer launches (0/1), 1 if the shape has a row in the table
 * (0: fallback rules). */
int kb_tile_plan(int k, int inC, int outC, int32_t plan[6]);
/* Number of rows of the tile table; row i as rows[i*8 .. i*8+7] = k, inC, outC, then the plan fields of kb_tile_plan in
 * order (without the last).  Fills at most cap rows. */
int kb_tile_table(int32_t* rows, int cap, int32_t* count);

/* Self-test of the failure path of the bounded device-side waits (no counterpart in the reference): on the handle's
 * stream a kernel waits limitNs nanoseconds (at most 1e9) on a barrier that nothing arrives at, gives up and records a
 * status code, exactly as a convolution kernel does when one of its waits runs out.  The call then synchronises and
 * returns the resulting error (non-zero, "a device-side wait timed out ..."); the handle stays usable. */
int kb_selftest_wait_timeout(kb_handle* h, unsigned long long limitNs);

/* Replaces NeuralNet::isUsingFP16 (nninterface.h:88): returns the precision in *precision. */
int kb_handle_precision(const kb_handle* h, int* precision);

/* Replaces the device part of NeuralNet::getOutput (nninterface.h:117-123; cudabackend.cpp:3556-3795):
 * host buffers in, host buffers out, synchronous.
 *   spatial  [n][nnYLen][nnXLen][inC] fp32 NHWC, as filled by NNEvaluator (not yet symmetrised)
 *   global   [n][inGlobalC] fp32
 *   symmetry [n] values 0..7 (SymmetryHelpers, nninputs.cpp:529-597) or NULL for identity; applied to the
 *            inputs on the device and inverted on policy/ownership outputs
 * Outputs are raw logits (nninterface.h:116); any output pointer may be NULL:
 *   policy [n][nnYLen*nnXLen][policyC], policyPass [n][policyC], value [n][valueC],
 *   scoreValue [n][scoreValueC], ownership [n][nnYLen*nnXLen]. */
int kb_forward_host(
  kb_handle* h, int n, const float* spatial, const float* global, const int32_t* symmetry,
  float* policy, float* policyPass, float* value, float* scoreValue, float* ownership);

/* The same for nets with an SGF metadata encoder (NNResultBuf::rowMetaBuf / hasRowMeta, nninputs.h; eigenbackend.cpp
 * 2458-2471): meta is [n][metaChannels] fp32 and must be non-NULL exactly when the model has the encoder. */
int kb_forward_host_meta(
  kb_handle* h, int n, const float* spatial, const float* global, const float* meta, const int32_t* symmetry,
  float* policy, float* policyPass, float* value, float* scoreValue, float* ownership);
int kb_upload_inputs_meta(kb_handle* h, int n, const float* spatial, const float* global, const float* meta, const int32_t* symmetry);

/* The three stages of kb_forward_host as separate calls, for measurements with the inputs
 * already resident in device memory: upload (host->device, asynchronous on the handle's stream),
 * run (all kernels of one forward pass), download (device->host, synchronises). */
int kb_upload_inputs(kb_handle* h, int n, const float* spatial, const float* global, const int32_t* symmetry);
int kb_forward_resident(kb_handle* h, int n);
int kb_download_outputs(
  kb_handle* h, int n, float* policy, float* policyPass, float* value, float* scoreValue, float* ownership);

/* Runs `iters` forward passes on resident inputs and returns the mean device time of one pass
 * in milliseconds, measured with CUDA events on the handle's stream. */
int kb_time_forward_resident(kb_handle* h, int n, int iters, float* msPerIter);

/* Times `steps` forward passes one by one: before each pass `flushBytes` bytes of scratch device memory are
 * overwritten (0 = no flush) so that the pass starts with a cold L2; the pass itself is bracketed by its own pair
 * of CUDA events on the handle's stream.  msEach[i] receives the device time of pass i in milliseconds. */
int kb_time_forward_steps(kb_handle* h, int n, int steps, size_t flushBytes, float* msEach);

/* Per-kernel-class device timing.  When enabled, every launch of kb_forward_resident is bracketed
 * by CUDA events on the handle's stream; kb_profile_read synchronises and returns, for up to `cap`
 * kernel classes, the class name (<=47 chars), number of launches and total milliseconds since the
 * last reset, and per-class algorithmic flops and bytes summed over those launches. */
typedef struct kb_profile_entry {
  char name[48];
  int64_t launches;
  double ms;
  double flops;
  double bytes;
} kb_profile_entry;
int kb_profile_enable(kb_handle* h, int enabled);
int kb_profile_reset(kb_handle* h);
int kb_profile_read(kb_handle* h, kb_profile_entry* entries, int cap, int* count);

/* Number of kernel launches one forward pass of batch n issues (for the harness's launch count). */
int kb_launches_per_forward(const kb_handle* h, int n, int* launches);

/* Trunk output after the final norm+activation, [n][nnYLen*nnXLen][trunkC] fp32 (debugging aid;
 * mirrors the reference's DEBUG_INTERMEDIATE_VALUES dumps, cudabackend.cpp:46). */
int kb_debug_read_trunk(kb_handle* h, int n, float* trunkOut);

/* Page-locked host memory for the staging buffers the caller fills (replaces the plain `new float[]`
 * staging of the reference's InputBuffers, cudabackend.cpp:3438-3551): copies from/to such memory are
 * asynchronous DMA transfers.  Usable from any thread, with or without a bound device. */
int kb_host_alloc(size_t bytes, void** out);
void kb_host_free(void* p);

/* Replaces NeuralNet::testEvaluateConv / BatchNorm / ResidualBlock / GlobalPoolingResidualBlock
 * (nninterface.h:134-180).  The blob holds one CONV, BN, BLOCK_ORDINARY or BLOCK_GPOOL construct.
 * in [n][Y][X][inC] NHWC fp32, mask [n][Y][X] (may be NULL for CONV), out [n][Y][X][outC]. */
int kb_eval_layer(
  const void* blob, size_t nbytes, int device, int precision, int n, int nnXLen, int nnYLen,
  const float* in, const float* mask, float* out);

/* Convolution without any allocation.  (No counterpart in the reference: its backends allocate freely.)
 *
 * For callers that may not allocate device memory themselves or through this library: plug-ins living inside a
 * host application's memory pool, or latency-critical loops that cannot afford the locks and the implicit
 * synchronisation of cudaMalloc/cudaFree.  The caller passes DEVICE pointers it already owns; the working
 * memory the convolution needs (padded copies of input and output, re-ordered weights) is a fixed 2.4 MiB array
 * inside the library's device image, present on every GPU that loads the library until the process exits.
 *
 *   dIn      [n][nnYLen][nnXLen][inC] fp32 NHWC     dWeights [outC][inC][kY][kX] fp32 (ConvLayerDesc order, desc.h:23)
 *   dOut     [n][nnYLen][nnXLen][outC] fp32 NHWC    stream   a cudaStream_t (NULL = default stream)
 * Computes the same zero-padded stride-1 cross-correlation as kb_eval_layer does for a CONV record in fp32.
 * The kernels are enqueued on `stream`; the call returns without waiting for them.
 *
 * Limits (exceeding one is an error, nothing is launched): n*(nnYLen+1)*(nnXLen+1) rounded up to a multiple of 256 <= 4096 rows
 * (10 boards of 19x19), inC <= 64, outC <= 64, kernel at most 5x5 and odd.
 * The first call on each device looks up the array's device address (with that device current); make that
 * call before starting any stream capture.  All calls share the one array and it keeps the previous call's
 * contents: two calls whose kernels overlap on the GPU (different streams, different threads) race on it.
 * The call itself performs no cudaMalloc, cudaFree or other allocating routine. */
int kb_conv_noalloc(
  const float* dIn, const float* dWeights, float* dOut, int n, int nnXLen, int nnYLen, int inC, int outC, int kY, int kX,
  void* stream);
/* Message of the last kb_conv_noalloc failure on the calling thread. */
const char* kb_conv_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* KATAB200_H_ */
