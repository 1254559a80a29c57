/* CPU oracle for the KataGo neural-net forward pass.  TEST INFRASTRUCTURE ONLY:
 * the shipped library never links, loads or calls anything declared here.
 *
 * It restates, in plain fp32 C++ with direct convolutions, the arithmetic of the
 * reference's Eigen backend (cpp/neuralnet/eigenbackend.cpp), which the reference
 * treats as the source of truth for all other backends (cpp/tests/tests.h:96-100).
 * Parity is pinned by running the reference's own known-answer tests against it:
 * tests/testnn.cpp (layer vectors) and tests/tinymodel.cpp (whole-net vector); the
 * recipe in oracle/Makefile links the reference's unmodified test sources with
 * oracle/oraclebackend.cpp; its printouts on the reference's shipped nets agree with
 * the golden text files under cpp/tests/results.  The transformer blocks, the RMS norms
 * and the SGF metadata encoder have no vector in the reference's C++ tests: they are
 * pinned to the reference's own PyTorch definitions (python/katago/train/model_pytorch.py)
 * through model files written by the reference's unmodified exporter and the nets' fp32
 * outputs (tests/golden/make_torch_golden.py, tests/test_oracle_pins.py).  The
 * relative-position attention bias is an extension of this repository's blob and is
 * defined here: parity unpinned for that one piece.
 *
 * All tensors are fp32, NHWC: spatial[n][y][x][c].  Models arrive as the blob
 * described in include/kb_modelblob.h.  Every function returns 0 on success and
 * a non-zero code on failure, with a message available from ko_last_error().
 */
#ifndef KATA_ORACLE_H_
#define KATA_ORACLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ko_model ko_model;

/* Message of the last failure on the calling thread. */
const char* ko_last_error(void);

/* Parses a model blob for boards of nnXLen x nnYLen.  *out is NULL on failure. */
int ko_model_create(const void* blob, size_t nbytes, int nnXLen, int nnYLen, ko_model** out);
void ko_model_destroy(ko_model* m);

/* info[0..8] = modelVersion, inC, inGlobalC, policyC, valueC, scoreValueC, ownershipC, trunkC, numBlocks */
int ko_model_info(const ko_model* m, int32_t info[9]);

/* Whole-network forward (eigenbackend.cpp:2150-2204 Model::apply).
 * spatial [n][Y][X][inC], global [n][inGlobalC].
 * Outputs (any may be NULL): policy [n][Y*X][policyC], policyPass [n][policyC],
 * value [n][valueC], scoreValue [n][scoreValueC], ownership [n][Y*X],
 * trunkOut [n][Y*X][trunkC] = trunk after the final norm+activation. */
int ko_forward(
  const ko_model* m, int n, const float* spatial, const float* global,
  float* policy, float* policyPass, float* value, float* scoreValue, float* ownership,
  float* trunkOut);

/* The same for nets with an SGF metadata encoder (eigenbackend.cpp:2458-2471): meta [n][metaChannels], non-NULL exactly
 * for those nets. */
int ko_forward_meta(
  const ko_model* m, int n, const float* spatial, const float* global, const float* meta,
  float* policy, float* policyPass, float* value, float* scoreValue, float* ownership,
  float* trunkOut);
/* The residual stream of the trunk (eigenbackend.cpp:1851-1936) as it enters each block and as it leaves the last one:
 * streams [numBlocks + 1][n][Y*X][trunkC].  Lets a test hand one block of a deep net its true input. */
int ko_trunk_streams(const ko_model* m, int n, const float* spatial, const float* global, const float* meta, float* streams);
/* ModelDesc::numInputMetaChannels (0 without the encoder). */
int ko_model_meta_channels(const ko_model* m, int32_t* channels);

/* Single-layer evaluation for the reference's layer tests (nninterface.h:134-180).
 * The blob holds exactly one CONV, BN, BLOCK_ORDINARY or BLOCK_GPOOL construct.
 * in [n][Y][X][inC], mask [n][Y][X] (ignored for CONV), out [n][Y][X][outC]. */
int ko_eval_layer(
  const void* blob, size_t nbytes, int n, int nnXLen, int nnYLen,
  const float* in, const float* mask, float* out);

/* Storage emulation, for measuring precision floors only (no counterpart in the reference): rounds the chosen tensors
 * of the convolutional blocks to storageType (0 = off, 1 = fp16, 2 = bf16) where a reduced-precision backend stores
 * them, all arithmetic staying fp32.  KO_EMU_CONV_INPUTS: every convolution's input (the activated tensors that feed
 * the matrix units, the pooling layers' inputs and the sums stored ahead of a per-board bias); KO_EMU_STREAMS: the residual streams as the
 * next update reads them.  Weights are rounded by the caller (in
 * the blob).  Process-wide; set it before a forward pass, never during one. */
#define KO_EMU_CONV_INPUTS 1
#define KO_EMU_STREAMS 2
int ko_set_storage_emulation(int storageType, int flags);

/* Number of OpenMP threads the oracle will use (for reporting CPU baselines). */
int ko_num_threads(void);
/* Sets the number of OpenMP threads for forward passes started by the calling thread from now on (an OpenMP runtime
 * that another library initialised first may have fixed it at 1 from the environment). */
int ko_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
