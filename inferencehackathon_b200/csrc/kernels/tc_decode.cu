// Single-token linear layers on the tensor cores (tcgen05 / TMEM) with fused epilogues: the decode hot path.
//
// At one token a linear layer is a pure weight stream, so everything here serves HBM:
//  * weights are stored pre-tiled and pre-swizzled (see IhbTcDecArgs), a stage is ONE contiguous 32 KB bulk
//    copy (a thread gets a bulk copy accepted only every ~0.3 us whatever its size, so copies must be large
//    and two producer warps alternate);
//  * the activation row is written once per work unit into a resident shared-memory operand (row 0 of an
//    8-row swizzle group; the second 8-row group of the N = 16 tile aliases the first through a zero group
//    stride), so no per-stage activation copy exists;
//  * e4m3 products never pass through CUDA cores: the MMA reads both operands from shared memory; the epilogue
//    warps only fold each 128-wide K block's partial sum with scale_w * scale_x.
// Epilogues: store; all-reduce push + residual + RMSNorm (+ re-quantised activation row for the next layer);
// argmax; SwiGLU + re-quantisation. Units (row tile x K split x routing slot) that feed one output tile meet in
// an fp32 workspace and the last to arrive adds them in a fixed order.
//
// The reference runs these layers as SIMT GEMVs (kernels/k1_attn_prologue.cu:205-238,
// kernels/k5_experts.cu:91-149) or as cuBLASLt GEMMs padded to M = 16 followed by separate glue kernels
// (kernels/gemm_engine.cuh:48-192).
#include "tc_common.cuh"
#include "tails.cuh"

namespace ihb {

constexpr int TD_PRODUCERS = 2;
constexpr int TD_MMA_WARP = 2;      // warps 0-1: producers, warp 2: MMA + TMEM allocation, warp 3: idle
constexpr int TD_THREADS = 256;     // warps 4-7: epilogue (TMEM lane quarter = warp % 4)
constexpr int TD_NT = 16;           // MMA N (one real token column)
constexpr int TD_BBLK = 1024;       // bytes of the activation operand per K block (one 8-row swizzle group)
constexpr uint32_t TD_BSTRIDE = 0;  // group stride of the activation descriptor: rows 8-15 alias rows 0-7

struct TdSmem {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[8];
  uint64_t tmem_empty[8];
  uint64_t bready[2];
  uint32_t tmem_base;
  int abort_flag;
  int last_flag;
  int sel_e[IHB_MAX_TOPK];
  float sel_w[IHB_MAX_TOPK];
  float red_f[8];
  unsigned long long red_u[8];
};

struct TdUnit {
  int tile, member, row0, slot, kb0, kb1;
};

__device__ __forceinline__ TdUnit td_unit(const IhbTcDecArgs& a, int u, int nkb_total) {
  TdUnit un;
  const int s = u % a.ks;
  const int rest = u / a.ks;
  const int base = nkb_total / a.ks, rem = nkb_total % a.ks;
  un.kb0 = s * base + min(s, rem);
  un.kb1 = un.kb0 + base + (s < rem ? 1 : 0);
  const int rtiles = (a.rows + TC_BM - 1) / TC_BM;
  if (a.mode == IHB_TC_LINEAR) {
    un.tile = rest; un.slot = 0; un.member = s; un.row0 = rest * TC_BM;
  } else if (a.mode == IHB_TC_GATEUP) {
    un.slot = rest / rtiles;
    un.tile = rest; un.member = s; un.row0 = (rest % rtiles) * TC_BM;
  } else {
    un.slot = rest % a.top_k;
    un.tile = rest / a.top_k;
    un.member = un.slot * a.ks + s;
    un.row0 = un.tile * TC_BM;
  }
  return un;
}

// Byte offset of K block `kb` of the row tile starting at `row0` of matrix `mat` in the tiled weight layout.
__device__ __forceinline__ size_t td_weight_offset(int mat, int row0, int kb, int rows_p8, int nkb_total) {
  const int rows_t = min(TC_BM, rows_p8 - row0);
  return (static_cast<size_t>(mat) * rows_p8 + row0) * nkb_total * TC_BKB + static_cast<size_t>(kb) * rows_t * TC_BKB;
}

#include "tc_decode_body.inc"

}  // namespace ihb

#include "tc_decode_host.inc"
