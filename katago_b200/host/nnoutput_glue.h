/* Row unpacking shared by the backends that implement the reference's
 * NeuralNet::getOutput contract (cpp/neuralnet/nninterface.h:102-123).
 *
 * unpackRow : raw network outputs of one row -> NNOutput fields, following the reference's
 *             CPU backend (neuralnet/eigenbackend.cpp:2527-2615): policy-optimism blend on
 *             policy channels 0/1, inverse symmetry for policy and ownership, pass logit at
 *             index X*Y, value logits, score-value fields by model version.
 */
#ifndef KATAGO_B200_HOST_NNOUTPUT_GLUE_H_
#define KATAGO_B200_HOST_NNOUTPUT_GLUE_H_

#include "neuralnet/nninputs.h"
#include "neuralnet/nneval.h"
#include "neuralnet/modelversion.h"

namespace kbhost {

struct NetDims {
  int modelVersion;
  int nnXLen;
  int nnYLen;
  int numSpatialFeatures;
  int numGlobalFeatures;
  int numPolicyChannels;
  int numValueChannels;
  int numScoreValueChannels;
};

inline NetDims makeNetDims(const ModelDesc& m, int nnXLen, int nnYLen) {
  NetDims d;
  d.modelVersion = m.modelVersion;
  d.nnXLen = nnXLen;
  d.nnYLen = nnYLen;
  d.numSpatialFeatures = m.numInputChannels;
  d.numGlobalFeatures = m.numInputGlobalChannels;
  d.numPolicyChannels = m.numPolicyChannels;
  d.numValueChannels = m.numValueChannels;
  d.numScoreValueChannels = m.numScoreValueChannels;
  if(NNModelVersion::getNumSpatialFeatures(m.modelVersion) != m.numInputChannels ||
     NNModelVersion::getNumGlobalFeatures(m.modelVersion) != m.numInputGlobalChannels)
    throw StringError("backend: model input channel counts do not match its model version");
  if(m.numValueChannels != 3 || m.numOwnershipChannels != 1)
    throw StringError("backend: unexpected number of value or ownership channels");
  return d;
}

// policy: [S][policyC] of this row; policyPass: [policyC]; value: [3]; scoreValue: [scoreValueC]; ownership: [S].
inline void unpackRow(
  const NetDims& d, const NNResultBuf* buf, NNOutput* output,
  const float* policy, const float* policyPass, const float* value, const float* scoreValue, const float* ownership) {
  const int S = d.nnXLen * d.nnYLen;
  const int Pc = d.numPolicyChannels;
  if(output->nnXLen != d.nnXLen || output->nnYLen != d.nnYLen)
    throw StringError("backend: NNOutput board size does not match the compute handle");

  float tmp[NNPos::MAX_NN_POLICY_SIZE];
  if(Pc == 2 || (Pc == 4 && d.modelVersion >= 16)) {
    const float optimism = (float)buf->policyOptimism;
    for(int i = 0; i < S; i++) {
      const float p = policy[(size_t)i * Pc];
      const float pOpt = policy[(size_t)i * Pc + 1];
      tmp[i] = p + (pOpt - p) * optimism;
    }
    SymmetryHelpers::copyOutputsWithSymmetry(tmp, output->policyProbs, 1, d.nnYLen, d.nnXLen, buf->symmetry);
    output->policyProbs[S] = policyPass[0] + (policyPass[1] - policyPass[0]) * optimism;
  }
  else if(Pc == 1) {
    SymmetryHelpers::copyOutputsWithSymmetry(policy, output->policyProbs, 1, d.nnYLen, d.nnXLen, buf->symmetry);
    output->policyProbs[S] = policyPass[0];
  }
  else {
    throw StringError("backend: unsupported number of policy channels");
  }

  output->whiteWinProb = value[0];
  output->whiteLossProb = value[1];
  output->whiteNoResultProb = value[2];

  if(output->whiteOwnerMap != NULL)
    SymmetryHelpers::copyOutputsWithSymmetry(ownership, output->whiteOwnerMap, 1, d.nnYLen, d.nnXLen, buf->symmetry);

  const int Sv = d.numScoreValueChannels;
  if(d.modelVersion >= 9) {
    if(Sv != 6) throw StringError("backend: expected 6 score value channels");
    output->whiteScoreMean = scoreValue[0];
    output->whiteScoreMeanSq = scoreValue[1];
    output->whiteLead = scoreValue[2];
    output->varTimeLeft = scoreValue[3];
    output->shorttermWinlossError = scoreValue[4];
    output->shorttermScoreError = scoreValue[5];
  }
  else if(d.modelVersion >= 8) {
    if(Sv != 4) throw StringError("backend: expected 4 score value channels");
    output->whiteScoreMean = scoreValue[0];
    output->whiteScoreMeanSq = scoreValue[1];
    output->whiteLead = scoreValue[2];
    output->varTimeLeft = scoreValue[3];
    output->shorttermWinlossError = 0;
    output->shorttermScoreError = 0;
  }
  else if(d.modelVersion >= 4) {
    if(Sv != 2) throw StringError("backend: expected 2 score value channels");
    output->whiteScoreMean = scoreValue[0];
    output->whiteScoreMeanSq = scoreValue[1];
    output->whiteLead = output->whiteScoreMean;
    output->varTimeLeft = 0;
    output->shorttermWinlossError = 0;
    output->shorttermScoreError = 0;
  }
  else {
    if(Sv != 1) throw StringError("backend: expected 1 score value channel");
    output->whiteScoreMean = scoreValue[0];
    // Version 3 nets have no second-moment output: use the square of the mean.
    output->whiteScoreMeanSq = output->whiteScoreMean * output->whiteScoreMean;
    output->whiteLead = output->whiteScoreMean;
    output->varTimeLeft = 0;
    output->shorttermWinlossError = 0;
    output->shorttermScoreError = 0;
  }
}

}  // namespace kbhost

#endif
