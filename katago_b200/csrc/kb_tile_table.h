// Tile table of the tensor-core convolution kernels: what the reference's OpenCL backend finds with its autotuner at
// start-up (cpp/neuralnet/opencltuner.cpp) is a committed table here, one row per convolution shape of the networks
// this library is measured on, each chosen from measurements on B200.  Host-only code (no CUDA): the planner of
// kb_conv_tc.cu and the C ABI (kb_tile_plan) both read it.
//
// A row fixes, for a convolution k x k, inC -> outC (inC as the device sees it, i.e. padded to a multiple of 64):
//   BN        output channels per tile = N of the MMA (M is always 128 rows, K chunks are 64 channels)
//   pair      1: CTA pairs (cta_group::2, 256-row tiles, half a weight tile per CTA)
//   epiWarps  epilogue warps per TMEM lane quarter WITHOUT a residual / WITH a residual (2 = 8 warps, 3 = 12 warps)
//   chain     1: runs of such convolutions execute as one persistent multi-layer launch (3x3 only)
// Shapes without a row fall back to rules that reproduce what the rows were generalised from: BN = the largest
// multiple of 16 that divides outC (at most 256), pairs for 3x3 with BN = 256, 12 epilogue warps for 1x1 convolutions
// with a residual.
//
// The comments give the measurement behind each row: microseconds per launch at the batch of the configuration
// (CUDA events around every launch) and, where captured, the tensor-pipe utilisation ncu reports for that launch
// (sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed, on a reduced-depth net at the same batch).
#pragma once

namespace kb {

struct TileRow {
  int k, inC, outC;
  int BN, pair, epiWarps, epiWarpsRes, chain;
};

static const TileRow TILE_TABLE[] = {
  // ---- b18c384nbt, fp16, batch 256 (102 400 padded rows = 800 row tiles) ----
  // 3x3 192->192: N=192 61 us, N=96 93 us, N=64 130 us per launch (the cost of an MMA has a large part that does not shrink
  // with N); CTA pairs 5-10 % slower; 12 epilogue warps 5 % slower (they cost a weight slot).  ncu: tensor pipe 54.9 % of
  // the launch (50.1 % with a residual); in a chain of four 55 us per layer at 66 %.
  {3, 192, 192, 192, 0, 2, 2, 1},
  // 3x3 128->192 (last convolution of a gpool block, with residual): the tile of the row above; 57 us, tensor pipe 38.9 %
  {3, 128, 192, 192, 0, 2, 2, 1},
  // 3x3 64->384 (stem: 22 input planes padded to 64): two channel tiles, bound by its epilogue; 77 us, tensor pipe 27.6 %
  {3, 64, 384, 192, 0, 2, 2, 0},
  // 1x1 384->192 (opens a nested block; also the merged head convolution p1|g1|v1): N=192 41.5 us, N=96 44.0, N=64 57.1;
  // tensor pipe 17.7 %
  {1, 384, 192, 192, 0, 2, 2, 0},
  // 1x1 192->384 with residual (closes a nested block): N=192 64.1 us, N=128 78.8, N=96 74.9; 12 epilogue warps 67.8 us
  // against 76.4 with 8; tensor pipe 11.1 %.  Followed by a 384->192 it runs fused with it (kb_conv_fused.cu): 81.5 us
  // under ncu for the pair against 101.5, tensor pipe 17.3 %.
  {1, 192, 384, 192, 0, 2, 3, 0},
  // ---- b28c512nbt, bf16, batch 512 (204 800 padded rows) ----
  // 3x3 256->256: N=256 with CTA pairs 179 us (1199 TFLOP/s; ncu: tensor pipe 80 %, 75 % with a residual), without pairs
  // 3 % slower; multi-layer launches bring nothing at 10.8 rounds of tiles per layer (730 us for four against 4 x 180)
  {3, 256, 256, 256, 1, 2, 2, 0},
  {3, 192, 256, 256, 1, 2, 2, 0},   // last convolution of a gpool block
  {3, 64, 512, 256, 1, 2, 2, 0},    // stem: 191 us, tensor pipe 29.7 %
  {1, 512, 256, 256, 0, 3, 3, 0},   // 84 us, tensor pipe 31 % (also the merged head convolution: 73 us, 36 %); 12 epilogue warps 97 -> 95 us
  // with residual: 180 us, tensor pipe 14 % with 8 epilogue warps; 12 warps (a tile's 8 units split 3 + 3 + 2) 212 -> 187 us
  // in the per-launch pass of the full net
  {1, 256, 512, 256, 0, 2, 3, 0},
  // ---- transformer 12 x (6 heads x 64, SwiGLU 1024), fp16, batch 128 (51 200 padded rows) ----
  // CTA pairs are slower for all four projections (Q|K|V 79 us against 66, attention output 41 against 36, up|gate 134
  // against 118, FFN down 68 against 66).
  // norm + Q|K|V: 66 us, tensor pipe 31 %; 83 us with the rotary embedding in its epilogue (which saves the attention
  // kernel 45 us).  N=128 with resident weights 91 us, N=96 114 us; 12 epilogue warps 84.5 us against 89.5 on one box,
  // 82.0 against 82.6 on another.
  {1, 384, 1152, 192, 0, 3, 2, 0},
  {1, 384, 384, 192, 0, 2, 3, 0},    // attention output with residual (records row sums): 38 us with 8 epilogue warps, 36 us with 12
  // norm + up|gate with the SwiGLU epilogue, which is the critical path (4 units of about 1650 cycles per warp and tile
  // against 5.8 k cycles of MMAs): 12 epilogue warps (8 units split 3 + 3 + 2) 105 us, 8 warps 121 us at 32 %; N=128 182 us
  {1, 384, 2048, 256, 0, 3, 2, 0},
  // FFN down with residual (records row sums): 62 us, 31 % under ncu; 72 -> 67 us with one barrier pair per K step, -> 62 us
  // with a fourth operand stage in place of a fourth residual slot (CUDA events, full net)
  {1, 1024, 384, 192, 0, 2, 2, 0},
};

inline const TileRow* tileTableLookup(int k, int inC, int outC) {
  for(const TileRow& r : TILE_TABLE)
    if(r.k == k && r.inC == inC && r.outC == outC) return &r;
  return nullptr;
}

// The plan for a shape: the table's row, or the fallback rules.  fromTable tells which.
inline TileRow tilePlanFor(int k, int inC, int outC, bool* fromTable = nullptr) {
  if(const TileRow* r = tileTableLookup(k, inC, outC)) {
    if(fromTable) *fromTable = true;
    return *r;
  }
  if(fromTable) *fromTable = false;
  TileRow r = {k, inC, outC, 0, 0, 2, 2, 0};
  for(int bn = 256; bn >= 16; bn -= 16)
    if(outC % bn == 0) { r.BN = bn; break; }
  r.pair = (k == 3 && r.BN == 256) ? 1 : 0;
  r.epiWarpsRes = (k == 1 && !r.pair && r.BN > 0 && (r.BN % 32) == 0) ? 3 : 2;
  r.chain = (k == 3 && !r.pair) ? 1 : 0;
  return r;
}

}  // namespace kb
