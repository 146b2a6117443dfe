// MoE expert kernels for one token (M = 1), sm_100a.
//
//   gateup:  act[s][j] = silu(<x, Wg[e_s][j]>) * <x, Wu[e_s][j]>        s = 0..top_k-1, e_s from the router tail
//   down:    y[o]      = sum_s w_s * <act[s], Wd[e_s][o]>               + fused all-reduce / residual / RMSNorm tail
//
// Both stream the selected experts' weight tiles through the bulk-copy ring of stream.cuh. The down projection
// gives each consumer warp one routing slot (its activation fragment stays in registers) and adds the slots in
// a fixed order in shared memory: no atomics, deterministic. The reference accumulates the eight experts with
// atomicAdd into a zeroed buffer (kernels/k5_experts.cu:125-149) and launches the all-reduce, residual add and
// norm as three more kernels (kernels/decode_step_tp8.cu:1100-1135).
#include "stream.cuh"
#include "api.h"
#include "tails.cuh"

namespace ihb {

template <int WT, int NI>
struct XSel;
template <int NI>
struct XSel<0, NI> { using type = XFragF16<NI>; };
template <int NI>
struct XSel<1, NI> { using type = XFragF32<NI>; };

// ---------------------------------------------------------------------------------------------------------------------
// gate/up + SwiGLU. Tile = R gate rows + R up rows of one routing slot. Stage layout:
//   [gate R rows][up R rows] ... pad ... [gate scale row 64 f32][up scale row 64 f32]
// ---------------------------------------------------------------------------------------------------------------------
template <int WT, int NI>
__global__ void __launch_bounds__(STREAM_THREADS, 1) moe_gateup_kernel(const IhbMoeArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int esize = (WT == 0) ? 1 : 2;
  const int row_bytes = a.H * esize;
  const int R = a.R_gu;
  const int stage_stride = ((2 * R * row_bytes + 127) & ~127) + 512;
  Ring ring = ring_setup(smem, a.S, stage_stride, tid, R);
  __syncthreads();
  const int tiles_per_slot = a.I / R;
  const int ntiles = a.top_k * tiles_per_slot;
  const int my_tiles = (static_cast<int>(blockIdx.x) < ntiles) ? (ntiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
  const size_t expert_bytes = static_cast<size_t>(2) * a.I * row_bytes;
  const int gu_nrb = (2 * a.I + a.gu_rb - 1) / a.gu_rb;
  bool ok = true;

  if (warp == NCW) {
    pdl_wait();   // expert ids come from the router kernel
    int my_e = 0;                              // lane s holds the local expert index of routing slot s
    if (lane < a.top_k) {
      my_e = ld_cg_i(a.sel_idx + lane) - a.expert0;
      if (my_e < 0 || my_e >= a.E_local) my_e = 0;   // not held here (expert parallel): rows are read but ignored
    }
    for (int it = 0; it < my_tiles && ok; ++it) {
      const int tile = blockIdx.x + it * gridDim.x;
      const int st = it % a.S;
      const unsigned ph = (it / a.S) & 1u;
      if (it >= a.S) ok = mbar_wait(&ring.empty[st], ph ^ 1u, a.err, ERR_MBAR_EMPTY_TIMEOUT);
      if (!ok) break;
      const int s = tile / tiles_per_slot;
      const int j0 = (tile % tiles_per_slot) * R;
      const int e = __shfl_sync(0xffffffffu, my_e, s);
      uint8_t* dst = ring.stages + static_cast<size_t>(st) * stage_stride;
      const uint8_t* wg = a.Wgu + e * expert_bytes + static_cast<size_t>(j0) * row_bytes;
      const uint8_t* wu = wg + static_cast<size_t>(a.I) * row_bytes;
      const uint32_t bytes = static_cast<uint32_t>(R) * row_bytes;
      if (lane == 0) {
        const uint32_t sbytes = (WT == 0) ? static_cast<uint32_t>(a.gu_nkb) * 4u : 0u;
        mbar_arrive_expect_tx(&ring.full[st], 2 * (bytes + sbytes));
        bulk_g2s(dst, wg, bytes, &ring.full[st]);
        bulk_g2s(dst + bytes, wu, bytes, &ring.full[st]);
        if (WT == 0) {
          const float* base = a.gu_scale + static_cast<size_t>(e) * gu_nrb * a.gu_nkb;
          bulk_g2s(dst + stage_stride - 512, base + static_cast<size_t>(j0 / a.gu_rb) * a.gu_nkb, sbytes,
                   &ring.full[st]);
          bulk_g2s(dst + stage_stride - 256, base + static_cast<size_t>((a.I + j0) / a.gu_rb) * a.gu_nkb, sbytes,
                   &ring.full[st]);
        }
      }
    }
    return;
  }

  pdl_wait();
  pdl_launch_dependents();
  const int celems = (WT == 0) ? 16 : 8;
  const int nchunks = a.H / celems;
  typename XSel<WT, NI>::type xf;
  xf.load(a.x, nchunks, lane);
  const int kb_shift = a.gu_kb_shift - 4;

  const int total_rows = my_tiles * R;      // row pairs dealt round-robin across tiles (see gemv.cu)
  for (int vr = warp; vr < total_rows && ok; vr += NCW) {
    const int it = vr / R;
    const int r = vr - it * R;
    const int tile = blockIdx.x + it * gridDim.x;
    const int st = it % a.S;
    const unsigned ph = (it / a.S) & 1u;
    ok = mbar_wait(&ring.full[st], ph, a.err, ERR_MBAR_FULL_TIMEOUT);
    if (!ok) break;
    const int s = tile / tiles_per_slot;
    const int j0 = (tile % tiles_per_slot) * R;
    const uint8_t* stg = ring.stages + static_cast<size_t>(st) * stage_stride;
    const float* sc = reinterpret_cast<const float*>(stg + stage_stride - 512);
    const uint8_t* gp = stg + static_cast<size_t>(r) * row_bytes;
    const uint8_t* up = gp + static_cast<size_t>(R) * row_bytes;
    float g, u;
    if constexpr (WT == 0) {
      g = row_dot_fp8<NI>(gp, xf, sc, 0, kb_shift, nchunks, lane);
      u = row_dot_fp8<NI>(up, xf, sc + 64, 0, kb_shift, nchunks, lane);
    } else {
      g = row_dot_bf16<NI>(gp, xf, nchunks, lane);
      u = row_dot_bf16<NI>(up, xf, nchunks, lane);
    }
    if (lane == 0) a.act[static_cast<size_t>(s) * a.I + j0 + r] = silu(g) * u;
    __syncwarp();
    if (lane == 0) mbar_arrive(&ring.empty[st]);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// down projection. Tile = R output rows x top_k slots. Stage layout:
//   [slot 0: R rows][slot 1: R rows] ... pad ... [scale row per slot, 64 f32 each]
// Warp w works on slot (w % top_k) and row group (w / top_k); a row is shared by G lanes.
// ---------------------------------------------------------------------------------------------------------------------
template <int WT, int NI>
__global__ void __launch_bounds__(STREAM_THREADS, 1) moe_down_kernel(const IhbMoeArgs a, const int G) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float red_f[NCW];
  __shared__ float part[2][IHB_MAX_TOPK][64];   // [tile parity][slot][row in tile]
  __shared__ int s_last;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int esize = (WT == 0) ? 1 : 2;
  const int row_bytes = a.I * esize;
  const int R = a.R_d;
  const int k = a.top_k;
  const int stage_stride = ((k * R * row_bytes + 127) & ~127) + k * 256;
  Ring ring = ring_setup(smem, a.S, stage_stride, tid, NCW);
  __syncthreads();
  const int ntiles = a.H / R;
  const int my_tiles = (static_cast<int>(blockIdx.x) < ntiles) ? (ntiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
  const size_t expert_bytes = static_cast<size_t>(a.H) * row_bytes;
  const int d_nrb = (a.H + a.d_rb - 1) / a.d_rb;
  bool ok = true;

  if (warp == NCW) {
    pdl_wait();   // expert ids: written two kernels back, visible once the previous kernel has passed its own wait
    int my_e = 0;
    if (lane < k) {
      my_e = ld_cg_i(a.sel_idx + lane) - a.expert0;
      if (my_e < 0 || my_e >= a.E_local) my_e = 0;
    }
    for (int it = 0; it < my_tiles && ok; ++it) {
      const int tile = blockIdx.x + it * gridDim.x;
      const int st = it % a.S;
      const unsigned ph = (it / a.S) & 1u;
      if (it >= a.S) ok = mbar_wait(&ring.empty[st], ph ^ 1u, a.err, ERR_MBAR_EMPTY_TIMEOUT);
      if (!ok) break;
      const int o0 = tile * R;
      uint8_t* dst = ring.stages + static_cast<size_t>(st) * stage_stride;
      const uint32_t bytes = static_cast<uint32_t>(R) * row_bytes;
      const uint32_t sbytes = (WT == 0) ? static_cast<uint32_t>(a.d_nkb) * 4u : 0u;
      if (lane == 0) mbar_arrive_expect_tx(&ring.full[st], k * (bytes + sbytes));
      __syncwarp();
      if (lane < k) {
        bulk_g2s(dst + lane * bytes, a.Wd + my_e * expert_bytes + static_cast<size_t>(o0) * row_bytes, bytes,
                 &ring.full[st]);
        if (WT == 0)
          bulk_g2s(dst + stage_stride - k * 256 + lane * 256,
                   a.d_scale + (static_cast<size_t>(my_e) * d_nrb + o0 / a.d_rb) * a.d_nkb, sbytes, &ring.full[st]);
      }
    }
    return;
  }

  pdl_wait();
  pdl_launch_dependents();
  const int celems = (WT == 0) ? 16 : 8;
  const int nchunks = a.I / celems;
  const int s = warp % k;                 // routing slot of this warp
  const int grp = warp / k, ngrp = NCW / k;
  const int rows_per_pass = 32 / G;       // rows a warp covers at once
  const int q = lane / G, g = lane % G;
  typename XSel<WT, NI>::type xf;
  xf.load(a.act + static_cast<size_t>(s) * a.I, nchunks, g, G);
  const int kb_shift = a.d_kb_shift - 4;
  int e_s = ld_cg_i(a.sel_idx + s) - a.expert0;
  const float w_s = (e_s >= 0 && e_s < a.E_local) ? ld_cg_f(a.sel_w + s) : 0.f;   // not held here -> contributes 0
  const int parity = (*a.comm.epoch) & 1u;

  for (int it = 0; it < my_tiles && ok; ++it) {
    const int tile = blockIdx.x + it * gridDim.x;
    const int st = it % a.S;
    const unsigned ph = (it / a.S) & 1u;
    ok = mbar_wait(&ring.full[st], ph, a.err, ERR_MBAR_FULL_TIMEOUT);
    if (!ok) break;
    const uint8_t* stg = ring.stages + static_cast<size_t>(st) * stage_stride;
    const float* sc = reinterpret_cast<const float*>(stg + stage_stride - k * 256) + s * 64;
    const uint8_t* slot_base = stg + static_cast<size_t>(s) * R * row_bytes;
    float (*pp)[64] = part[it & 1];
    for (int r0 = grp * rows_per_pass; r0 < R; r0 += ngrp * rows_per_pass) {
      const int r = r0 + q;
      float y;                    // R is a multiple of the rows one pass covers, so r < R for every lane
      const uint8_t* rowp = slot_base + static_cast<size_t>(r) * row_bytes;
      if constexpr (WT == 0) {
        y = group_dot_fp8<NI>(rowp, xf, sc, kb_shift, nchunks, g, G);
      } else {
        y = group_dot_bf16<NI>(rowp, xf, nchunks, g, G);
      }
      if (g == 0) pp[s][r] = y * w_s;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&ring.empty[st]);
    named_bar_sync(1, CONSUMER_THREADS);
    if (tid < R) {
      float y = 0.f;
      for (int ss = 0; ss < k; ++ss) y += pp[ss][tid];
      const int row = tile * R + tid;
      const IhbComm& cm = a.comm;
      const size_t off = (static_cast<size_t>(parity) * cm.nranks + cm.rank) * a.H + row;
      push_partial(cm, off, y);
    }
  }

  // last-CTA election and the all-reduce / residual / norm tail
  if (tid < 64) {   // the threads that pushed partials
    if (a.comm.nranks > 1) __threadfence_system(); else __threadfence();
  }
  named_bar_sync(1, CONSUMER_THREADS);
  if (tid == 0) {
    const unsigned old = atomicAdd(a.counter, 1u);
    s_last = (old == gridDim.x - 1);
    if (s_last) {
      *a.counter = 0u;
      __threadfence();
    }
  }
  named_bar_sync(1, CONSUMER_THREADS);
  if (!s_last) return;
  ArNormTail t{a.comm, a.H, 1, a.resid, a.gamma, a.xn_out, a.eps, a.err, nullptr, nullptr, 0};
  tail_ar_norm<CONSUMER_THREADS, 1>(t, tid, red_f);
}

static int num_sms() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

static void fill_cfg(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int grid, int smem, int use_pdl,
                     cudaStream_t stream) {
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(STREAM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl ? 1 : 0;
}

}  // namespace ihb

using namespace ihb;

extern "C" int ihb_moe_gateup(IhbMoeArgs* args, int use_pdl, cudaStream_t stream) {
  IhbMoeArgs a = *args;
  const int esize = a.wtype == IHB_W_FP8 ? 1 : 2;
  const int celems = a.wtype == IHB_W_FP8 ? 16 : 8;
  if (a.H % celems || a.top_k < 1 || a.top_k > IHB_MAX_TOPK) return cudaErrorInvalidValue;
  const int ni = (a.H / celems + 31) / 32;
  if (ni > 8) return cudaErrorInvalidValue;
  if (a.wtype == IHB_W_FP8 && (a.gu_nkb > 64 || (a.gu_nkb & 3) || a.gu_kb_shift < 4)) return cudaErrorInvalidValue;
  const int row_bytes = a.H * esize;
  const int sms = num_sms();
  if (a.R_gu <= 0) {
    int best_R = 1;
    float best_cost = 1e30f;
    for (int R = 64; R >= 1; R /= 2) {
      if (a.I % R) continue;
      if (R > 1 && 2 * R * row_bytes > 32768) continue;
      if (a.wtype == IHB_W_FP8 && (a.gu_rb % R) != 0) continue;
      const int tiles = a.top_k * (a.I / R);
      const float cost = static_cast<float>((tiles + sms - 1) / sms) * R * (1.f + 0.5f / R);
      if (cost < best_cost) { best_cost = cost; best_R = R; }
    }
    a.R_gu = best_R;
  }
  if (a.I % a.R_gu) return cudaErrorInvalidValue;
  if (a.wtype == IHB_W_FP8 && (a.gu_rb % a.R_gu)) return cudaErrorInvalidValue;
  const int stage_stride = ((2 * a.R_gu * row_bytes + 127) & ~127) + 512;
  if (a.S <= 0) {
    int S = (200 * 1024) / stage_stride;
    a.S = S > 12 ? 12 : S;
  }
  if (a.S < 2 || a.S > 12) return cudaErrorInvalidValue;
  const int smem = 256 + a.S * stage_stride;
  const int ntiles = a.top_k * (a.I / a.R_gu);
  int grid = a.grid > 0 ? a.grid : sms;
  if (grid > ntiles) grid = ntiles;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  fill_cfg(cfg, attr, grid, smem, use_pdl, stream);
  cudaError_t e;
#define GU(WT, NI)                                                                                               \
  do {                                                                                                           \
    e = cudaFuncSetAttribute(moe_gateup_kernel<WT, NI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);      \
    if (e != cudaSuccess) return e;                                                                              \
    return cudaLaunchKernelEx(&cfg, moe_gateup_kernel<WT, NI>, a);                                               \
  } while (0)
  const int nisel = ni <= 1 ? 1 : ni <= 2 ? 2 : ni <= 4 ? 4 : 8;
  if (a.wtype == IHB_W_FP8) {
    switch (nisel) { case 1: GU(0, 1); case 2: GU(0, 2); case 4: GU(0, 4); default: GU(0, 8); }
  } else {
    switch (nisel) { case 1: GU(1, 1); case 2: GU(1, 2); case 4: GU(1, 4); default: GU(1, 8); }
  }
#undef GU
}

extern "C" int ihb_moe_down(IhbMoeArgs* args, int use_pdl, cudaStream_t stream) {
  IhbMoeArgs a = *args;
  const int esize = a.wtype == IHB_W_FP8 ? 1 : 2;
  const int celems = a.wtype == IHB_W_FP8 ? 16 : 8;
  const int k = a.top_k;
  if (a.I % celems || k < 1 || k > IHB_MAX_TOPK || (NCW % k) != 0) return cudaErrorInvalidValue;
  if (a.wtype == IHB_W_FP8 && (a.d_nkb > 64 || (a.d_nkb & 3) || a.d_kb_shift < 4)) return cudaErrorInvalidValue;
  const int nchunks = a.I / celems;
  // lanes per row: smallest power of two G with ceil(nchunks / G) <= 4
  int G = 1;
  while (G < 32 && (nchunks + G - 1) / G > 4) G *= 2;
  const int ni = (nchunks + G - 1) / G;
  if (ni > 8) return cudaErrorInvalidValue;
  const int row_bytes = a.I * esize;
  const int sms = num_sms();
  const int ngrp = NCW / k;
  const int min_R = (32 / G) * ngrp;           // one pass of every warp
  if (a.R_d <= 0) {
    int R = 32768 / (k * row_bytes);
    if (R < 1) R = 1;
    int p = 1;
    while (p * 2 <= R) p *= 2;
    R = p;
    while (R > min_R && a.H / R < 3 * sms) R /= 2;
    if (R < min_R) R = min_R;
    if (R > 64) R = 64;
    a.R_d = R;
  }
  if (a.R_d > 64 || a.H % a.R_d) return cudaErrorInvalidValue;
  if (a.wtype == IHB_W_FP8 && (a.d_rb % a.R_d)) return cudaErrorInvalidValue;
  const int stage_stride = ((k * a.R_d * row_bytes + 127) & ~127) + k * 256;
  if (a.S <= 0) {
    int S = (200 * 1024) / stage_stride;
    a.S = S > 12 ? 12 : S;
  }
  if (a.S < 2 || a.S > 12) return cudaErrorInvalidValue;
  const int smem = 256 + a.S * stage_stride;
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  const int ntiles = a.H / a.R_d;
  int grid = a.grid > 0 ? a.grid : sms;
  if (grid > ntiles) grid = ntiles;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  fill_cfg(cfg, attr, grid, smem, use_pdl, stream);
  cudaError_t e;
#define DN(WT, NI)                                                                                               \
  do {                                                                                                           \
    e = cudaFuncSetAttribute(moe_down_kernel<WT, NI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);        \
    if (e != cudaSuccess) return e;                                                                              \
    return cudaLaunchKernelEx(&cfg, moe_down_kernel<WT, NI>, a, G);                                              \
  } while (0)
  const int nisel = ni <= 1 ? 1 : ni <= 2 ? 2 : ni <= 4 ? 4 : 8;
  if (a.wtype == IHB_W_FP8) {
    switch (nisel) { case 1: DN(0, 1); case 2: DN(0, 2); case 4: DN(0, 4); default: DN(0, 8); }
  } else {
    switch (nisel) { case 1: DN(1, 1); case 2: DN(1, 2); case 4: DN(1, 4); default: DN(1, 8); }
  }
#undef DN
}
