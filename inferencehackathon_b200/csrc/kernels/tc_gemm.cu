// Tensor-core linear layers for sm_100a: tcgen05.mma with TMEM accumulators, operands staged by TMA.
//
//   Y[t, r] = sum_k X[t, k] * W[r, k]        W: block-scaled e4m3 (128-wide K blocks) or bf16, K-major rows
//                                            X: e4m3 with one scale per token per 128 channels, or bf16
//
// The WEIGHT rows are the MMA's M dimension (128 rows per tile = the 128 TMEM lanes) and the TOKENS are N
// (16..128), so that one kernel serves single-token decode (N padded to 16), speculative verify windows and
// prefill chunks, and a token count far below 128 wastes nothing but idle tensor-core columns. Per K block of
// 128 bytes a stage holds a 128x128-byte weight tile and an Nx128-byte activation tile, both written by TMA
// with the 128-byte swizzle that the shared-memory matrix descriptors name; one thread issues four MMAs
// (K = 32 bytes each) per stage. For block-scaled fp8 every K block accumulates into its own TMEM buffer (two,
// ping-pong) and the epilogue warps fold it into fp32 registers with scale_w[row block, k block] *
// scale_x[token, k block]; bf16 accumulates the whole K range in TMEM.
//
// Work units are (row tile, K split[, routing slot]); when several units feed one output tile their partials
// go through a small fp32 workspace and the last unit to arrive adds them in a fixed order (deterministic).
//
// The reference reaches tensor cores only through cuBLASLt calls at M = 16 (kernels/gemm_engine.cuh:48-125)
// and one mma.sync prefill kernel (kernels/prefill_wgmma.cu:88-262).
#include <string.h>
#include "tc_common.cuh"
#include "tails.cuh"

namespace ihb {

constexpr int TC_PRODUCERS = 3;     // a thread gets one bulk/TMA copy accepted every ~0.3 us whatever its size, so
                                    // three producer warps take the stages round-robin
constexpr int TC_MMA_WARP = 3;
constexpr int TC_THREADS = 256;     // warps 0-2: TMA producers, warp 3: MMA + TMEM allocation, warps 4-7: epilogue

struct TcSmem {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[8];
  uint64_t tmem_empty[8];
  uint32_t tmem_base;
  int abort_flag;
  int last_flag;
  int sel_e[IHB_MAX_TOPK];       // local expert index per routing slot
  float sel_w[IHB_MAX_TOPK];
};

struct Unit {
  int tile;      // output tile index (mode 0: row tile; mode 1: slot * jtiles + jt; mode 2: row tile)
  int member;    // index of this unit among the units that add into the same tile
  int row0;      // first weight row of the tile (mode 1: j0 inside the expert's gate block)
  int slot;      // routing slot (modes 1, 2) else 0
  int kb0, kb1;  // K blocks [kb0, kb1)
  int e, tok0, ntok;   // local expert (grouped mode), first row of X, valid rows
  int orow0;           // first output row of the unit
};

constexpr int TC_GRP_SMEM = 1024;   // group-table entries kept in shared memory (16 KB); larger tables are read from global

__device__ __forceinline__ Unit decode_unit(const IhbTcArgs& a, int u, int nkb_total, const int4* grp_s) {
  Unit un;
  un.e = 0; un.tok0 = a.tok0; un.ntok = a.T; un.orow0 = 0;
  if (a.groups != nullptr) {
    const int rtiles = (a.rows + TC_BM - 1) / TC_BM;
    const int g = u / rtiles, tile = u - g * rtiles;
    // every role decodes every unit: from shared memory this costs a few cycles, from global a round trip per unit
    const int4 gr = grp_s != nullptr ? grp_s[g] : *reinterpret_cast<const int4*>(a.groups + 4 * g);
    un.e = gr.x; un.tok0 = gr.y; un.ntok = gr.z;
    un.tile = u; un.member = 0; un.row0 = tile * TC_BM; un.slot = 0; un.kb0 = 0; un.kb1 = nkb_total;
    un.orow0 = un.tok0;
    return un;
  }
  const int s = u % a.ks;
  int rest = u / a.ks;
  const int base = nkb_total / a.ks, rem = nkb_total % a.ks;
  un.kb0 = s * base + min(s, rem);
  un.kb1 = un.kb0 + base + (s < rem ? 1 : 0);
  if (a.mode == IHB_TC_LINEAR) {
    // several token tiles in one launch: a weight tile's units of all token tiles are neighbours, so that the tile is
    // fetched from HBM once and from L2 afterwards
    const int tt = a.tok_tiles > 1 ? rest % a.tok_tiles : 0;
    const int rt = a.tok_tiles > 1 ? rest / a.tok_tiles : rest;
    un.tile = rest; un.slot = 0; un.member = s; un.row0 = rt * TC_BM;
    if (a.tok_tiles > 1) {
      un.orow0 = tt * a.tok_tile;
      un.tok0 = a.tok0 + un.orow0;
      un.ntok = min(a.tok_tile, a.T - un.orow0);
    }
  } else if (a.mode == IHB_TC_GATEUP) {
    const int jtiles = (a.rows + TC_BM - 1) / TC_BM;      // rows = I
    un.slot = rest / jtiles;
    const int jt = rest % jtiles;
    un.tile = rest; un.member = s; un.row0 = jt * TC_BM;
  } else {   // DOWN: units ordered (tile, slot, split) so that a tile's members are contiguous
    un.slot = rest % a.top_k;
    un.tile = rest / a.top_k;
    un.member = un.slot * a.ks + s;
    un.row0 = un.tile * TC_BM;
  }
  return un;
}

// KIND 0 = block-scaled fp8, 1 = bf16. NT = token tile (MMA N). NA = A tiles per stage (2 for gate/up).
template <int KIND, int NT, int NA>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const IhbTcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  TcSmem& sh = *reinterpret_cast<TcSmem*>(smem);
  const int esize = (KIND == 0) ? 1 : 2;
  const int nkb_total = (a.K * esize + TC_BKB - 1) / TC_BKB;
  const int nslot_x = (a.mode == IHB_TC_DOWN) ? a.top_k : 1;
  const int grp_n = (a.groups != nullptr && a.max_groups <= TC_GRP_SMEM) ? a.max_groups : 0;
  const int grp_bytes = (grp_n * 16 + 1023) & ~1023;
  int4* grp_w = reinterpret_cast<int4*>(smem + 1024);                      // the group table (grouped mode)
  const int4* grp_s = grp_n > 0 ? grp_w : nullptr;
  float* xs_s = reinterpret_cast<float*>(smem + 1024 + grp_bytes);         // [nslot_x][nkb_total][NT] (fp8 only)
  const int xs_bytes = (KIND == 0) ? ((nslot_x * nkb_total * NT * 4 + 1023) & ~1023) : 0;
  uint8_t* stages = smem + 1024 + grp_bytes + xs_bytes;
  constexpr int B_BYTES = NT * TC_BKB;
  constexpr int STAGE_BYTES = NA * TC_A_BYTES + B_BYTES;
  const int S = a.S;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // With few token columns an MMA is over in a handful of cycles but its result takes a pipeline latency to
  // land, so MMAs chained on ONE accumulator run at latency, not throughput. The four K steps of a stage
  // therefore go to SUB = 4 separate accumulators (added up by the epilogue) when N is small.
#ifdef IHB_TC_SUB_WIDE
  constexpr int SUB = (NT <= 32) ? 4 : (NT == 64 ? (NA == 1 ? 4 : 2) : 2);
#else
  constexpr int SUB = (NT <= 32) ? 4 : 1;
#endif
  constexpr int BUF_COLS = NA * SUB * NT;
  // accumulator ring in tensor memory: up to 8 buffers (512 columns in total)
  constexpr int NBUF = (512 / BUF_COLS) >= 8 ? 8 : (512 / BUF_COLS);
  static_assert(NBUF >= 2, "need two accumulator buffers");
  constexpr uint32_t TMEM_COLS_NEEDED = NBUF * BUF_COLS;
  constexpr uint32_t TMEM_COLS = TMEM_COLS_NEEDED <= 32 ? 32 : TMEM_COLS_NEEDED <= 64 ? 64
                               : TMEM_COLS_NEEDED <= 128 ? 128 : TMEM_COLS_NEEDED <= 256 ? 256 : 512;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 1); }
    for (int b = 0; b < NBUF; ++b) { mbar_init(&sh.tmem_full[b], 1); mbar_init(&sh.tmem_empty[b], 4); }
    sh.abort_flag = 0;
    sh.last_flag = 0;
    fence_mbar_init();
  }
  if (warp == TC_MMA_WARP) tmem_alloc(&sh.tmem_base, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;
  volatile int* abort_flag = &sh.abort_flag;

  // Everything below reads outputs of earlier kernels (activations, expert ids).
  pdl_wait();
  pdl_launch_dependents();
  if (a.mode != IHB_TC_LINEAR && a.groups == nullptr && tid < a.top_k) {
    int e = ld_cg_i(a.sel_idx + tid) - a.expert0;
    const bool here = (e >= 0 && e < a.n_experts);
    sh.sel_e[tid] = here ? e : 0;
    sh.sel_w[tid] = here ? ld_cg_f(a.sel_w + tid) : 0.f;
  }
  if (grp_n > 0) {
    const int ng = min(ld_cg_i(a.n_groups), grp_n);
    for (int i = tid; i < ng; i += TC_THREADS) grp_w[i] = *reinterpret_cast<const int4*>(a.groups + 4 * i);
  }
  if (a.x_rows1) {
    // single-token mode copies only row 0 of each activation tile: clear the other rows once
    for (int i = tid; i < S * (B_BYTES / 16); i += TC_THREADS) {
      const int st = i / (B_BYTES / 16), o = i % (B_BYTES / 16);
      *reinterpret_cast<uint4*>(stages + static_cast<size_t>(st) * STAGE_BYTES + NA * TC_A_BYTES + o * 16) = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async_smem();
  }
  if (KIND == 0 && warp >= 4 && a.groups == nullptr && a.tok_tiles <= 1) {
    // activation scales for every K block: global layout [slot][kb][T], padded here to NT columns
    const int n = nslot_x * nkb_total * NT;
    for (int i = tid - 128; i < n; i += 128) {
      const int col = i % NT, r = i / NT;
      xs_s[i] = (col < a.T) ? ld_cg_f(a.xscale + static_cast<size_t>(r) * a.T_total + a.tok0 + col) : 0.f;
    }
  }
  __syncthreads();

  const int total_units = a.groups != nullptr ? ld_cg_i(a.n_groups) * ((a.rows + TC_BM - 1) / TC_BM) : a.n_units;
  const uint32_t idesc = (1u << 4) | (KIND == 1 ? ((1u << 7) | (1u << 10)) : 0u) |
                         (static_cast<uint32_t>(NT >> 3) << 17) | (static_cast<uint32_t>(TC_BM >> 4) << 24);
  const int kx = TC_BKB / esize;     // K elements per block (tensor-map coordinate units)
  const int rows_p8 = (a.rows + 7) & ~7;

  if (warp < TC_PRODUCERS) {
    // =============================== TMA producers: warp p feeds the stages with g % 3 == p ============================
    // The whole warp runs the loop and lane 0 issues (see tc_common.cuh: the copies want warp-uniform operands).
    const unsigned leader = lane == 0 ? 1u : 0u;
    int g = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
      const Unit un = decode_unit(a, u, nkb_total, grp_s);
      const int e = (a.mode == IHB_TC_LINEAR) ? 0 : (a.groups != nullptr ? un.e : sh.sel_e[un.slot]);
      for (int kb = un.kb0; kb < un.kb1; ++kb, ++g) {
        if (g % TC_PRODUCERS != warp) continue;
        const int st = g % S;
        if (g >= S) ok = tc_wait(&sh.empty[st], ((g / S) & 1u) ^ 1u, abort_flag, a.err, ERR_MBAR_EMPTY_TIMEOUT);
        if (!ok) break;
        uint8_t* sA = stages + static_cast<size_t>(st) * STAGE_BYTES;
        uint8_t* sB = sA + NA * TC_A_BYTES;
        if (a.tiled) {
          // Pre-tiled weights: [matrix][k block][rows padded to 8][128 B], already in the swizzled order, so a
          // tile of this K block is ONE contiguous run of up to 16 KB.
          const int rows_here = min(TC_BM, rows_p8 - un.row0);
          const uint32_t abytes = static_cast<uint32_t>(rows_here) * TC_BKB;
          const uint32_t bbytes = a.x_rows1 ? TC_BKB : B_BYTES;
          mbar_arrive_expect_tx_if(leader, &sh.full[st], NA * abytes + bbytes);
          const size_t panel = static_cast<size_t>(rows_p8) * TC_BKB;                 // one K block of one matrix
          const size_t mat = (a.mode == IHB_TC_GATEUP) ? static_cast<size_t>(e) * 2 : static_cast<size_t>(e);
          const uint8_t* src = reinterpret_cast<const uint8_t*>(a.W) + (mat * nkb_total + kb) * panel +
                               static_cast<size_t>(un.row0) * TC_BKB;
          bulk_g2s_if(leader, sA, src, abytes, &sh.full[st]);
          if (NA == 2) bulk_g2s_if(leader, sA + TC_A_BYTES, src + static_cast<size_t>(nkb_total) * panel, abytes, &sh.full[st]);
          if (a.x_rows1) {
            // one token: row 0 of the (pre-zeroed) activation tile; the swizzle of row 0 is the identity
            const uint8_t* xs = reinterpret_cast<const uint8_t*>(a.X) +
                                (static_cast<size_t>(a.mode == IHB_TC_DOWN ? un.slot : 0) * nkb_total + kb) * TC_BKB;
            bulk_g2s_if(leader, sB, xs, TC_BKB, &sh.full[st]);
          } else if (a.mode == IHB_TC_DOWN) {
            tma_load_3d_if(leader, sB, &tmB, kb * kx, un.tok0, un.slot, &sh.full[st]);
          } else {
            tma_load_2d_if(leader, sB, &tmB, kb * kx, un.tok0, &sh.full[st]);
          }
        } else {
          mbar_arrive_expect_tx_if(leader, &sh.full[st], STAGE_BYTES);
          if (a.mode == IHB_TC_LINEAR) {
            tma_load_2d_if(leader, sA, &tmA, kb * kx, un.row0, &sh.full[st]);
            tma_load_2d_if(leader, sB, &tmB, kb * kx, un.tok0, &sh.full[st]);
          } else if (a.mode == IHB_TC_GATEUP) {
            tma_load_4d_if(leader, sA, &tmA, kb * kx, un.row0, 0, e, &sh.full[st]);
            if (NA == 2) tma_load_4d_if(leader, sA + TC_A_BYTES, &tmA, kb * kx, un.row0, 1, e, &sh.full[st]);
            tma_load_2d_if(leader, sB, &tmB, kb * kx, un.tok0, &sh.full[st]);
          } else {
            tma_load_3d_if(leader, sA, &tmA, kb * kx, un.row0, e, &sh.full[st]);
            tma_load_3d_if(leader, sB, &tmB, kb * kx, un.tok0, un.slot, &sh.full[st]);
          }
        }
      }
    }
  } else if (warp == TC_MMA_WARP) {
    // =============================== MMA issuer ========================================================================
    // One thread, inside a branch: measured with a one-CTA micro-kernel, this form issues a 128 x 128 x 16 MMA every 64
    // cycles (the tensor rate) with descriptors that change per instruction, while a warp-uniform loop with a predicated
    // tcgen05.mma needed 118-180.
    if (lane == 0) {
      int g = 0, ui = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++ui) {
        const Unit un = decode_unit(a, u, nkb_total, grp_s);
        for (int kb = un.kb0; kb < un.kb1 && ok; ++kb, ++g) {
          const int st = g % S;
          ok = tc_wait(&sh.full[st], (g / S) & 1u, abort_flag, a.err, ERR_MBAR_FULL_TIMEOUT);
          if (!ok) break;
          const int j = (KIND == 0) ? g : ui;            // accumulator use counter
          const int b = j % NBUF;
          if ((KIND == 0 || kb == un.kb0) && j >= NBUF) {
            ok = tc_wait(&sh.tmem_empty[b], ((j / NBUF) & 1u) ^ 1u, abort_flag, a.err, ERR_TMEM_TIMEOUT);
            if (!ok) break;
          }
          tc_fence_after();
          const uint8_t* sA = stages + static_cast<size_t>(st) * STAGE_BYTES;
          const uint64_t bdesc = smem_desc_sw128(sA + NA * TC_A_BYTES);
#pragma unroll
          for (int ai = 0; ai < NA; ++ai) {
            const uint64_t adesc = smem_desc_sw128(sA + ai * TC_A_BYTES);
#pragma unroll
            for (int k = 0; k < TC_BKB / 32; ++k) {
              const int sub = k % SUB;
              const uint32_t d = tmem_base + static_cast<uint32_t>(b * BUF_COLS + (ai * SUB + sub) * NT);
              const uint32_t accf = (KIND == 0) ? (k >= SUB) : (kb > un.kb0 || k >= SUB);
              tc_mma<KIND>(d, adesc + 2 * k, bdesc + 2 * k, idesc, accf);   // +32 bytes of K per step
            }
          }
          tc_commit(&sh.empty[st]);                      // stage reusable once these MMAs have read it
          if (KIND == 0 || kb == un.kb1 - 1) tc_commit(&sh.tmem_full[b]);
        }
      }
    }
  } else {
    // =============================== epilogue warps (TMEM lane quarter = warp % 4) =================================================
    const int quarter = warp & 3;
    const int r_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const int etid = tid - 128;                        // 0..127
    int g = 0, ui = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++ui) {
      const Unit un = decode_unit(a, u, nkb_total, grp_s);
      const int e = (a.mode == IHB_TC_LINEAR) ? 0 : (a.groups != nullptr ? un.e : sh.sel_e[un.slot]);
      if (KIND == 0 && (a.groups != nullptr || a.tok_tiles > 1)) {
        // grouped / token-tiled mode: the activation scales of this unit's tokens (the previous unit's readers are done: barrier)
        named_bar_sync(2, 128);
        for (int i = etid; i < nkb_total * NT; i += 128) {
          const int col = i % NT, r = i / NT;
          xs_s[i] = (col < un.ntok) ? ld_cg_f(a.xscale + static_cast<size_t>(r) * a.T_total + un.tok0 + col) : 0.f;
        }
        named_bar_sync(2, 128);
      }
      float acc[NA][NT];
#pragma unroll
      for (int ai = 0; ai < NA; ++ai)
#pragma unroll
        for (int n = 0; n < NT; ++n) acc[ai][n] = 0.f;
      if (KIND == 0) {
        // weight scale rows of this thread's weight row(s)
        const float* wsp[NA];
#pragma unroll
        for (int ai = 0; ai < NA; ++ai) {
          int wr = un.row0 + r_in_tile;
          if (wr >= a.rows) wr = a.rows - 1;
          if (a.mode == IHB_TC_GATEUP) wr += ai * a.rows;      // up rows follow the gate rows
          wsp[ai] = a.wscale + (static_cast<size_t>(e) * a.nrb + wr / a.rb) * a.nkb_stride;
        }
        float ws_next[NA];
#pragma unroll
        for (int ai = 0; ai < NA; ++ai) ws_next[ai] = __ldg(wsp[ai] + un.kb0);
        const float* xsl = xs_s + static_cast<size_t>(a.mode == IHB_TC_DOWN ? un.slot : 0) * nkb_total * NT;
        for (int kb = un.kb0; kb < un.kb1 && ok; ++kb, ++g) {
          float ws[NA];
#pragma unroll
          for (int ai = 0; ai < NA; ++ai) {
            ws[ai] = ws_next[ai];
            if (kb + 1 < un.kb1) ws_next[ai] = __ldg(wsp[ai] + kb + 1);
          }
          const int b = g % NBUF;
          ok = tc_wait(&sh.tmem_full[b], (g / NBUF) & 1u, abort_flag, a.err, ERR_TMEM_TIMEOUT);
          if (!ok) break;
          tc_fence_after();
          const float* xk = xsl + static_cast<size_t>(kb) * NT;
#pragma unroll
          for (int ai = 0; ai < NA; ++ai) {
#pragma unroll
            for (int c = 0; c < NT; c += 16) {
              float d[16];
              tmem_ld16(lane_addr + static_cast<uint32_t>(b * BUF_COLS + ai * SUB * NT + c), d);
#pragma unroll
              for (int sub = 1; sub < SUB; ++sub) {
                float d2[16];
                tmem_ld16(lane_addr + static_cast<uint32_t>(b * BUF_COLS + (ai * SUB + sub) * NT + c), d2);
#pragma unroll
                for (int n = 0; n < 16; ++n) d[n] += d2[n];
              }
#pragma unroll
              for (int n = 0; n < 16; ++n) acc[ai][c + n] = fmaf(d[n], ws[ai] * xk[c + n], acc[ai][c + n]);
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sh.tmem_empty[b]);
        }
      } else {
        g += un.kb1 - un.kb0;
        const int b = ui % NBUF;
        ok = tc_wait(&sh.tmem_full[b], (ui / NBUF) & 1u, abort_flag, a.err, ERR_TMEM_TIMEOUT);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int ai = 0; ai < NA; ++ai)
#pragma unroll
            for (int c = 0; c < NT; c += 16) {
              tmem_ld16(lane_addr + static_cast<uint32_t>(b * BUF_COLS + ai * SUB * NT + c), &acc[ai][c]);
#pragma unroll
              for (int sub = 1; sub < SUB; ++sub) {
                float d2[16];
                tmem_ld16(lane_addr + static_cast<uint32_t>(b * BUF_COLS + (ai * SUB + sub) * NT + c), d2);
#pragma unroll
                for (int n = 0; n < 16; ++n) acc[ai][c + n] += d2[n];
              }
            }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sh.tmem_empty[b]);
        }
      }
      if (!ok) break;

      // ---- combine the units that feed this output tile -------------------------------------------------------------------
      const int members = a.groups != nullptr ? 1 : ((a.mode == IHB_TC_DOWN) ? a.top_k * a.ks : a.ks);
      const float wslot = (a.mode == IHB_TC_DOWN && a.groups == nullptr) ? sh.sel_w[un.slot] : 1.f;
      bool finisher = true;
      if (members > 1) {
        float* part = a.partial + (static_cast<size_t>(un.tile) * members + un.member) * (NA * NT * TC_BM);
#pragma unroll
        for (int ai = 0; ai < NA; ++ai)
#pragma unroll
          for (int n = 0; n < NT; ++n)
            if (n < un.ntok) part[(ai * NT + n) * TC_BM + r_in_tile] = acc[ai][n] * wslot;
        __threadfence();
        named_bar_sync(2, 128);
        if (etid == 0) {
          const unsigned old = atomicAdd(a.tile_counters + un.tile, 1u);
          const int last = (old == static_cast<unsigned>(members) - 1u);
          if (last) { a.tile_counters[un.tile] = 0u; __threadfence(); }
          sh.last_flag = last;
        }
        named_bar_sync(2, 128);
        finisher = sh.last_flag != 0;
        if (finisher) {
          // members in a fixed order (deterministic sums); all token columns of one member are read together, so
          // that a member costs one memory round trip instead of one per column
          const float* p0 = a.partial + static_cast<size_t>(un.tile) * members * (NA * NT * TC_BM);
#pragma unroll
          for (int ai = 0; ai < NA; ++ai)
#pragma unroll
            for (int n = 0; n < NT; ++n) acc[ai][n] = 0.f;
          for (int mbr = 0; mbr < members; ++mbr) {
            const float* pm = p0 + static_cast<size_t>(mbr) * NA * NT * TC_BM + r_in_tile;
#pragma unroll
            for (int ai = 0; ai < NA; ++ai)
#pragma unroll
              for (int n = 0; n < NT; ++n)
                if (n < un.ntok) acc[ai][n] += ld_cg_f(pm + static_cast<size_t>(ai * NT + n) * TC_BM);
          }
        }
        named_bar_sync(2, 128);      // last_flag is rewritten by the next unit
      } else if (a.mode == IHB_TC_DOWN) {
#pragma unroll
        for (int n = 0; n < NT; ++n) acc[0][n] *= wslot;
      }
      if (!finisher) continue;

      // ---- epilogue on the finished tile: this thread owns weight row `row` for every token ----------------------------
      const int row = un.row0 + r_in_tile;
      if (a.mode == IHB_TC_GATEUP) {
        // SwiGLU; `out` is [slot][T][I] fp32
        if (row < a.rows) {
#pragma unroll
          for (int n = 0; n < NT; ++n)
            if (n < un.ntok) {
              const size_t orow = a.groups != nullptr ? static_cast<size_t>(un.orow0 + n) : static_cast<size_t>(un.slot) * a.T + n;
              a.out[orow * a.rows + row] = silu(acc[0][n]) * acc[NA - 1][n];
            }
        }
      } else {
        if (row < a.rows) {
#pragma unroll
          for (int n = 0; n < NT; ++n)
            if (n < un.ntok) a.out[static_cast<size_t>(un.orow0 + n) * a.out_stride + row] = acc[0][n];
        }
      }
    }
  }

  // ---- teardown: every role arrives here, also after a time-out ------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == TC_MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host side ------------------------------------------------------------------------------------------------------------------

// The tensor-map encoder is the only driver-API call of this library. It is resolved through the runtime at first
// use instead of being linked, so that the library also loads on a machine without a GPU driver (build checks).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

static CUresult encode_map(CUtensorMap* tm, int is_fp8, void* base, int rank, const cuuint64_t* dims,
                           const cuuint64_t* strides_bytes, const cuuint32_t* box) {
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return CUDA_ERROR_NOT_FOUND;
  return enc(tm, is_fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, base, dims, strides_bytes,
             box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

template <int KIND, int NT, int NA>
static cudaError_t launch_tc(const CUtensorMap& tmA, const CUtensorMap& tmB, const IhbTcArgs& a, int grid, int smem,
                             int use_pdl, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(tc_gemm_kernel<KIND, NT, NA>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, tc_gemm_kernel<KIND, NT, NA>, tmA, tmB, a);
}

}  // namespace ihb

using namespace ihb;

extern "C" size_t ihb_tc_partial_floats(const IhbTcArgs* a) {
  const int tiles_rows = (a->rows + TC_BM - 1) / TC_BM;
  const int tt = (a->mode == IHB_TC_LINEAR && a->tok_tiles > 1) ? a->tok_tiles : 1;
  const int tiles = (a->mode == IHB_TC_GATEUP ? a->top_k * tiles_rows : tiles_rows) * tt;
  const int members = a->mode == IHB_TC_DOWN ? a->top_k * a->ks : a->ks;
  const int na = a->mode == IHB_TC_GATEUP ? 2 : 1;
  const int t1 = tt > 1 ? a->tok_tile : a->T;
  const int nt = t1 <= 16 ? 16 : t1 <= 32 ? 32 : t1 <= 64 ? 64 : 128;
  return members > 1 ? static_cast<size_t>(tiles) * members * na * nt * TC_BM : 0;
}

// Picks the K split so that the grid has about two waves of units, encodes the tensor maps and launches.
extern "C" int ihb_tc_gemm(IhbTcArgs* args, int use_pdl, cudaStream_t stream) {
  IhbTcArgs a = *args;
  const int is_fp8 = a.wtype == IHB_W_FP8;
  const int esize = is_fp8 ? 1 : 2;
  const int grouped = a.groups != nullptr;
  if (grouped && (a.mode == IHB_TC_LINEAR || a.n_groups == nullptr || a.max_groups < 1 || a.tiled || a.x_rows1)) return cudaErrorInvalidValue;
  if (grouped) { a.top_k = 1; a.ks = 1; a.tok0 = 0; }
  // LINEAR over more than one token tile: tok_tiles tiles of tok_tile (16, 32, 64 or 128) tokens cover the T tokens
  if (a.tok_tiles > 1) {
    if (a.mode != IHB_TC_LINEAR || grouped || a.tiled || a.x_rows1) return cudaErrorInvalidValue;
    if ((a.tok_tile != 16 && a.tok_tile != 32 && a.tok_tile != 64 && a.tok_tile != 128) || a.T < 1 ||
        a.T > a.tok_tile * a.tok_tiles || a.T <= a.tok_tile * (a.tok_tiles - 1)) return cudaErrorInvalidValue;
  } else {
    a.tok_tiles = 1;
    if (a.T < 1 || a.T > 128) return cudaErrorInvalidValue;
  }
  if (a.rows < 1 || a.K < 1 || (a.K * esize) % 16) return cudaErrorInvalidValue;
  if (is_fp8 && (a.rb < 1 || a.wscale == nullptr || a.xscale == nullptr)) return cudaErrorInvalidValue;
  if (a.mode != IHB_TC_LINEAR && (a.top_k < 1 || a.top_k > IHB_MAX_TOPK)) return cudaErrorInvalidValue;
  const int t_tile = a.tok_tiles > 1 ? a.tok_tile : a.T;
  const int nt = t_tile <= 16 ? 16 : t_tile <= 32 ? 32 : t_tile <= 64 ? 64 : 128;
  if (a.mode == IHB_TC_GATEUP && nt > 64) return cudaErrorInvalidValue;   // two accumulators per token column
  const int na = a.mode == IHB_TC_GATEUP ? 2 : 1;
  const int nkb_total = (a.K * esize + TC_BKB - 1) / TC_BKB;
  const int tiles_rows = (a.rows + TC_BM - 1) / TC_BM;
  int sms = 148;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int base_units = a.mode == IHB_TC_LINEAR ? tiles_rows * a.tok_tiles : a.top_k * tiles_rows;
  if (a.ks <= 0) {
    int ks = (2 * sms + base_units - 1) / base_units;
    if (ks > nkb_total) ks = nkb_total;
    if (ks > 16) ks = 16;
    if (ks < 1) ks = 1;
    a.ks = ks;
  }
  if (a.ks > nkb_total) a.ks = nkb_total;
  a.n_units = grouped ? a.max_groups * tiles_rows : base_units * a.ks;
  const int members = a.mode == IHB_TC_DOWN ? a.top_k * a.ks : a.ks;
  if (members > 1 && (a.partial == nullptr || a.tile_counters == nullptr)) return cudaErrorInvalidValue;

  // tensor maps -----------------------------------------------------------------------------------------------------------
  alignas(64) CUtensorMap tmA, tmB;
  const cuuint64_t Kd = static_cast<cuuint64_t>(a.K);
  const cuuint64_t rowb = Kd * esize;
  const cuuint32_t kbox = TC_BKB / esize;
  CUresult r;
  memset(&tmA, 0, sizeof(tmA));
  memset(&tmB, 0, sizeof(tmB));
  if (a.tiled) {
    r = CUDA_SUCCESS;
  } else if (a.mode == IHB_TC_LINEAR) {
    cuuint64_t dims[2] = {Kd, static_cast<cuuint64_t>(a.rows)};
    cuuint64_t str[1] = {rowb};
    cuuint32_t box[2] = {kbox, TC_BM};
    r = encode_map(&tmA, is_fp8, const_cast<void*>(a.W), 2, dims, str, box);
  } else if (a.mode == IHB_TC_GATEUP) {       // [E][2][I][K]
    cuuint64_t dims[4] = {Kd, static_cast<cuuint64_t>(a.rows), 2, static_cast<cuuint64_t>(a.n_experts)};
    cuuint64_t str[3] = {rowb, rowb * a.rows, rowb * a.rows * 2};
    cuuint32_t box[4] = {kbox, TC_BM, 1, 1};
    r = encode_map(&tmA, is_fp8, const_cast<void*>(a.W), 4, dims, str, box);
  } else {                                    // [E][H][I]
    cuuint64_t dims[3] = {Kd, static_cast<cuuint64_t>(a.rows), static_cast<cuuint64_t>(a.n_experts)};
    cuuint64_t str[2] = {rowb, rowb * a.rows};
    cuuint32_t box[3] = {kbox, TC_BM, 1};
    r = encode_map(&tmA, is_fp8, const_cast<void*>(a.W), 3, dims, str, box);
  }
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  if (a.x_rows1) {
    if (a.T != 1 || !a.tiled) return cudaErrorInvalidValue;
    r = CUDA_SUCCESS;
  } else if (a.mode == IHB_TC_DOWN) {                // X: [top_k][T][K]
    cuuint64_t dims[3] = {Kd, static_cast<cuuint64_t>(a.T_total), static_cast<cuuint64_t>(a.top_k)};
    cuuint64_t str[2] = {rowb, rowb * a.T_total};
    cuuint32_t box[3] = {kbox, static_cast<cuuint32_t>(nt), 1};
    r = encode_map(&tmB, is_fp8, const_cast<void*>(a.X), 3, dims, str, box);
  } else {
    cuuint64_t dims[2] = {Kd, static_cast<cuuint64_t>(a.T_total)};
    cuuint64_t str[1] = {rowb};
    cuuint32_t box[2] = {kbox, static_cast<cuuint32_t>(nt)};
    r = encode_map(&tmB, is_fp8, const_cast<void*>(a.X), 2, dims, str, box);
  }
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;

  // shared memory ------------------------------------------------------------------------------------------------------------
  const int nslot_x = a.mode == IHB_TC_DOWN ? a.top_k : 1;
  const int xs_bytes = is_fp8 ? ((nslot_x * nkb_total * nt * 4 + 1023) & ~1023) : 0;
  const int stage_bytes = na * TC_A_BYTES + nt * TC_BKB;
  const int grp_bytes = (grouped && a.max_groups <= TC_GRP_SMEM) ? ((a.max_groups * 16 + 1023) & ~1023) : 0;
  int S = (200 * 1024 - 2048 - xs_bytes - grp_bytes) / stage_bytes;
  if (S > 8) S = 8;
  if (a.S > 0 && a.S < S) S = a.S;
  // With fewer stages than producer warps, the warp that refills a stage for the second time could pass the stage's
  // "empty" wait before the warp that refills it for the first time has loaded it (an mbarrier wait on the phase after
  // next succeeds at once): two arrivals on one "full" phase. From three stages up each warp's own earlier waits rule
  // that out.
  if (S < TC_PRODUCERS) return cudaErrorInvalidValue;
  a.S = S;
  const int smem = 1024 /*align slack*/ + 1024 + grp_bytes + xs_bytes + S * stage_bytes;
  int grid = a.grid > 0 ? a.grid : sms;
  if (grid > a.n_units) grid = a.n_units;

#define TC_GO(KIND, NT, NA) return launch_tc<KIND, NT, NA>(tmA, tmB, a, grid, smem, use_pdl, stream)
  if (is_fp8) {
    if (na == 1) {
      switch (nt) { case 16: TC_GO(0, 16, 1); case 32: TC_GO(0, 32, 1); case 64: TC_GO(0, 64, 1); default: TC_GO(0, 128, 1); }
    } else {
      switch (nt) { case 16: TC_GO(0, 16, 2); case 32: TC_GO(0, 32, 2); default: TC_GO(0, 64, 2); }
    }
  } else {
    if (na == 1) {
      switch (nt) { case 16: TC_GO(1, 16, 1); case 32: TC_GO(1, 32, 1); case 64: TC_GO(1, 64, 1); default: TC_GO(1, 128, 1); }
    } else {
      switch (nt) { case 16: TC_GO(1, 16, 2); case 32: TC_GO(1, 32, 2); default: TC_GO(1, 64, 2); }
    }
  }
#undef TC_GO
}
