// Decode GEMV (M = 1) with fused epilogues, sm_100a.
//
//   y[rows] = W[rows, K] . x[K]      W: block-scaled e4m3 or bf16, K-major rows; x: fp32 from the previous kernel
//
// Epilogues (the last CTA to finish runs a "tail" so that no second launch is needed):
//   STORE     y -> out                                      (QKV projection, logits for sampling)
//   ROUTER    y = router logits; tail: softmax, top-k, renormalise -> expert ids + weights
//   ARGMAX    per-CTA (max, arg); tail: global argmax -> next token, position counter += 1
//   AR_NORM   y is this rank's PARTIAL o_proj / down output: it is pushed into slot [rank] of a symmetric
//             buffer on EVERY GPU (one `multimem.st` per value through NVSwitch, or per-peer stores), one
//             cross-GPU arrive/wait, then the tail sums the slots in rank order (bitwise identical on all
//             ranks), adds the residual, applies the next RMSNorm and leaves the normed vector for the next
//             kernel. This replaces the reference's GEMV -> separate 1-block NVLS all-reduce kernel ->
//             residual/norm kernel chain (kernels/decode_step_tp8.cu:1093-1135, kernels/nvls_engine.cuh:160-200).
//
// With programmatic dependent launch the producer warp starts streaming weights before the previous kernel has
// finished; only the activation load waits for it.
#include "stream.cuh"
#include "api.h"
#include "tails.cuh"

namespace ihb {

template <int WT, int NI>
struct XFragSel;
template <int NI>
struct XFragSel<0, NI> { using type = XFragF16<NI>; };
template <int NI>
struct XFragSel<1, NI> { using type = XFragF32<NI>; };

// Router tail (one warp): softmax over E logits, top-k (ties -> lowest id), renormalise.
__device__ void tail_router(const IhbGemvArgs& a, int lane) {
  const int E = a.rows;
  constexpr int MAXPER = 8;   // E <= 256
  float v[MAXPER];
  float m = -INFINITY;
#pragma unroll
  for (int j = 0; j < MAXPER; ++j) {
    const int e = lane + 32 * j;
    v[j] = -INFINITY;
    if (e < E) {
      if (a.ks > 1) {           // K-split partial logits, added in slice order (identical on every rank)
        float s = 0.f;
        for (int h = 0; h < a.ks; ++h) s += ld_cg_f(a.router_partial + h * E + e);
        v[j] = s;
        a.out[e] = s;
      } else {
        v[j] = ld_cg_f(a.out + e);
      }
    }
    m = fmaxf(m, v[j]);
  }
  m = warp_max(m);
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < MAXPER; ++j) {
    v[j] = (lane + 32 * j < E) ? __expf(v[j] - m) : -1.f;   // probabilities are > 0; -1 marks "absent/taken"
    if (v[j] > 0.f) s += v[j];
  }
  s = warp_sum(s);
  float wsum = 0.f;
  float myw = 0.f;
  int myid = 0;
  for (int k = 0; k < a.top_k; ++k) {
    float bv = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < MAXPER; ++j) {
      const int e = lane + 32 * j;
      if (v[j] > bv) { bv = v[j]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((bi & 31) == lane) {
#pragma unroll
      for (int j = 0; j < MAXPER; ++j)
        if (lane + 32 * j == bi) v[j] = -1.f;
    }
    const float p = bv / s;
    wsum += p;
    if (lane == k) { myw = p; myid = bi; }
  }
  if (lane < a.top_k) {
    a.sel_idx[lane] = myid;
    a.sel_w[lane] = a.renorm ? myw / wsum : myw;
  }
}

// ---- the kernel ----------------------------------------------------------------------------------------------------

template <int WT, int NI, int EPI>
__global__ void __launch_bounds__(STREAM_THREADS, 1) gemv_kernel(const IhbGemvArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float red_f[NCW];
  __shared__ unsigned long long red_u[NCW];
  __shared__ int s_last;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int esize = (WT == 0) ? 1 : 2;
  const int row_bytes = a.K * esize;
  const int tile_bytes_full = a.R * row_bytes;
  const int stage_stride = ((tile_bytes_full + 127) & ~127) + 256;     // + scale row (<= 64 floats)
  const int vrows_per_tile = a.R * a.ks;            // one arrival on `empty` per (virtual) row consumed
  Ring ring = ring_setup(smem, a.S, stage_stride, tid, vrows_per_tile);
  __syncthreads();
  const int ntiles = (a.rows + a.R - 1) / a.R;
  const int my_tiles = (static_cast<int>(blockIdx.x) < ntiles) ? (ntiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
  bool ok = true;

  if (warp == NCW) {
    // ------------------------------- producer warp -----------------------------------------------------------
    for (int it = 0; it < my_tiles && ok; ++it) {
      const int tile = blockIdx.x + it * gridDim.x;
      const int st = it % a.S;
      const unsigned ph = (it / a.S) & 1u;
      if (it >= a.S) ok = mbar_wait(&ring.empty[st], ph ^ 1u, a.err, ERR_MBAR_EMPTY_TIMEOUT);
      if (!ok) break;
      const int row0 = tile * a.R;
      const int nrows = min(a.R, a.rows - row0);
      uint8_t* dst = ring.stages + static_cast<size_t>(st) * stage_stride;
      const uint32_t bytes = static_cast<uint32_t>(nrows) * row_bytes;
      if (lane == 0) {
        // weights and (fp8) the row block's scale row both arrive by bulk copy: the producer never waits on a load
        const uint32_t sbytes = (WT == 0) ? static_cast<uint32_t>(a.nkb) * 4u : 0u;
        mbar_arrive_expect_tx(&ring.full[st], bytes + sbytes);
        bulk_g2s(dst, a.W + static_cast<size_t>(row0) * row_bytes, bytes, &ring.full[st]);
        if (WT == 0)
          bulk_g2s(dst + stage_stride - 256, a.wscale + static_cast<size_t>(row0 / a.rb) * a.nkb, sbytes,
                   &ring.full[st]);
      }
    }
    // Error path: a wait above ran out after IHB_LOCAL_WAIT_NS, far longer than any copy takes, so nothing
    // issued by this warp is still in flight when it leaves.
    return;
  }

  // --------------------------------- consumer warps -----------------------------------------------------------------
  pdl_wait();
  pdl_launch_dependents();
  const int Kv = a.K / a.ks;                         // virtual row length (elements)
  const int celems = (WT == 0) ? 16 : 8;
  const int nchunks = Kv / celems;
  const int h = warp % a.ks;                         // K-slice of this warp (ks divides NCW)
  typename XFragSel<WT, NI>::type xf;
  xf.load(a.x + h * Kv, nchunks, lane);
  const int kb_shift = a.kb_shift - 4;               // scale block width in 16-element chunks (log2)
  const int chunk0 = h * nchunks;

  int parity = 0;
  if (EPI == IHB_EPI_AR_NORM) parity = (*a.comm.epoch) & 1u;
  unsigned long long best = 0ull;
  // Rows are dealt to the warps round-robin ACROSS tiles, so that short tiles (few rows) still keep all eight
  // warps busy, each on its own stage of the ring.
  const int total_vrows = my_tiles * vrows_per_tile;
  for (int vr = warp; vr < total_vrows && ok; vr += NCW) {
    const int it = vr / vrows_per_tile;
    const int v = vr - it * vrows_per_tile;
    const int tile = blockIdx.x + it * gridDim.x;
    const int st = it % a.S;
    const unsigned ph = (it / a.S) & 1u;
    ok = mbar_wait(&ring.full[st], ph, a.err, ERR_MBAR_FULL_TIMEOUT);
    if (!ok) break;
    const int row0 = tile * a.R;
    const int nrows = min(a.R, a.rows - row0);
    const uint8_t* stg = ring.stages + static_cast<size_t>(st) * stage_stride;
    const float* sc = reinterpret_cast<const float*>(stg + stage_stride - 256);
    const int r = v / a.ks;
    if (r < nrows) {
      const uint8_t* rowp = stg + static_cast<size_t>(r) * row_bytes + static_cast<size_t>(h) * Kv * esize;
      float y;
      if constexpr (WT == 0) {
        y = row_dot_fp8<NI>(rowp, xf, sc, chunk0, kb_shift, nchunks, lane);
      } else {
        y = row_dot_bf16<NI>(rowp, xf, nchunks, lane);
      }
      const int row = row0 + r;
      if (lane == 0) {
        if (EPI == IHB_EPI_ROUTER && a.ks > 1) {
          a.router_partial[h * a.rows + row] = y;
        } else if (EPI == IHB_EPI_STORE || EPI == IHB_EPI_ROUTER) {
          a.out[row] = y;
        } else if (EPI == IHB_EPI_ARGMAX) {
          const unsigned long long p = pack_max(y, static_cast<unsigned>(row));
          best = p > best ? p : best;
          if (a.out != nullptr) a.out[row] = y;
        } else {   // AR_NORM: push the partial into slot (rank, h) on every GPU
          const IhbComm& cm = a.comm;
          const size_t off = (static_cast<size_t>(parity) * cm.nranks * a.ks + cm.rank * a.ks + h) * a.rows + row;
          push_partial(cm, off, y);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&ring.empty[st]);
  }

  if (EPI == IHB_EPI_STORE) return;

  // ------------------------------------ last-CTA election and tail ------------------------------------------------------
  if (EPI == IHB_EPI_ARGMAX) {
    if (lane == 0) red_u[warp] = best;
  }
  if (lane == 0) {
    if (EPI == IHB_EPI_AR_NORM && a.comm.nranks > 1) __threadfence_system(); else __threadfence();
  }
  named_bar_sync(1, CONSUMER_THREADS);
  if (tid == 0) {
    if (EPI == IHB_EPI_ARGMAX) {
      unsigned long long b = red_u[0];
#pragma unroll
      for (int w = 1; w < NCW; ++w) b = red_u[w] > b ? red_u[w] : b;
      a.argmax_partial[blockIdx.x] = b;
      __threadfence();
    }
    const unsigned old = atomicAdd(a.counter, 1u);
    s_last = (old == gridDim.x - 1);
    if (s_last) {
      *a.counter = 0u;          // ready for the next launch (stream order / pdl_wait keeps it apart)
      __threadfence();
    }
  }
  named_bar_sync(1, CONSUMER_THREADS);
  if (!s_last) return;
  if (EPI == IHB_EPI_AR_NORM) {
    ArNormTail t{a.comm, a.rows, a.ks, a.resid, a.gamma, a.xn_out, a.eps, a.err, nullptr, nullptr, 0};
    tail_ar_norm<CONSUMER_THREADS, 1>(t, tid, red_f);
  }
  if (EPI == IHB_EPI_ROUTER) { if (warp == 0) tail_router(a, lane); }
  if (EPI == IHB_EPI_ARGMAX) {
    ArgmaxTail t{a.comm, a.argmax_partial, static_cast<int>(gridDim.x), a.vocab0, a.cur_token, a.pos, a.token_ring,
                 a.token_ring_size, a.forced, a.n_forced, a.err};
    tail_argmax<CONSUMER_THREADS, 1>(t, tid, red_u);
  }
}

template <int WT, int NI>
static cudaError_t launch_epi(const IhbGemvArgs& a, const cudaLaunchConfig_t& cfg) {
  switch (a.epi) {
    case IHB_EPI_STORE:   return cudaLaunchKernelEx(&cfg, gemv_kernel<WT, NI, IHB_EPI_STORE>, a);
    case IHB_EPI_ROUTER:  return cudaLaunchKernelEx(&cfg, gemv_kernel<WT, NI, IHB_EPI_ROUTER>, a);
    case IHB_EPI_ARGMAX:  return cudaLaunchKernelEx(&cfg, gemv_kernel<WT, NI, IHB_EPI_ARGMAX>, a);
    case IHB_EPI_AR_NORM: return cudaLaunchKernelEx(&cfg, gemv_kernel<WT, NI, IHB_EPI_AR_NORM>, a);
  }
  return cudaErrorInvalidValue;
}

template <int WT, int NI>
static cudaError_t set_smem(int epi, int bytes) {
  const void* f = nullptr;
  switch (epi) {
    case IHB_EPI_STORE:   f = reinterpret_cast<const void*>(gemv_kernel<WT, NI, IHB_EPI_STORE>); break;
    case IHB_EPI_ROUTER:  f = reinterpret_cast<const void*>(gemv_kernel<WT, NI, IHB_EPI_ROUTER>); break;
    case IHB_EPI_ARGMAX:  f = reinterpret_cast<const void*>(gemv_kernel<WT, NI, IHB_EPI_ARGMAX>); break;
    case IHB_EPI_AR_NORM: f = reinterpret_cast<const void*>(gemv_kernel<WT, NI, IHB_EPI_AR_NORM>); break;
  }
  return cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

}  // namespace ihb

using namespace ihb;

// Host entry. Picks the template instance from the weight type and the per-lane chunk count, fills in the tile
// height / stage count when the caller left them 0, and launches on `stream` (optionally with the programmatic
// dependent launch attribute). Returns a cudaError_t value.
extern "C" int ihb_gemv(IhbGemvArgs* args, int use_pdl, cudaStream_t stream) {
  IhbGemvArgs a = *args;
  const int esize = a.wtype == IHB_W_FP8 ? 1 : 2;
  const int celems = a.wtype == IHB_W_FP8 ? 16 : 8;
  if (a.ks < 1) a.ks = 1;
  if (a.K % (celems * a.ks) != 0 || (NCW % a.ks) != 0 || a.rows <= 0) return cudaErrorInvalidValue;
  if (a.ks > 1 && a.epi != IHB_EPI_AR_NORM && !(a.epi == IHB_EPI_ROUTER && a.router_partial != nullptr)) return cudaErrorInvalidValue;
  const int nchunks = a.K / a.ks / celems;
  const int ni = (nchunks + 31) / 32;
  if (ni > 16) return cudaErrorInvalidValue;
  if (a.wtype == IHB_W_FP8) {
    if (a.kb_shift < 4 || a.nkb > 64 || (a.nkb & 3) || a.rb <= 0) return cudaErrorInvalidValue;   // scale rows: 16-byte multiples
  }
  const int row_bytes = a.K * esize;
  int sms = 148;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  if (a.R <= 0) {
    // tile height: power of two, tile <= 32 KB, minimising the rows on the busiest CTA (ceil(tiles / SMs) * R)
    // with a mild preference for taller tiles (fewer barrier round trips per byte)
    int best_R = 1;
    float best_cost = 1e30f;
    for (int R = 64; R >= 1; R /= 2) {
      if (R > 1 && R * row_bytes > 32768) continue;
      if (a.wtype == IHB_W_FP8 && (a.rb % R) != 0) continue;
      const int tiles = (a.rows + R - 1) / R;
      const float cost = static_cast<float>((tiles + sms - 1) / sms) * R * (1.f + 0.5f / R);
      if (cost < best_cost) { best_cost = cost; best_R = R; }
    }
    a.R = best_R;
  }
  if (a.wtype == IHB_W_FP8 && (a.rb % a.R) != 0) return cudaErrorInvalidValue;
  const int stage_stride = ((a.R * row_bytes + 127) & ~127) + 256;
  if (a.S <= 0) {
    int S = (200 * 1024) / stage_stride;
    a.S = S > 12 ? 12 : S;
  }
  if (a.S < 2 || a.S > 12) return cudaErrorInvalidValue;
  const int smem_bytes = 256 + a.S * stage_stride;
  if (smem_bytes > 227 * 1024) return cudaErrorInvalidValue;
  const int ntiles = (a.rows + a.R - 1) / a.R;
  int grid = a.grid > 0 ? a.grid : sms;
  if (grid > ntiles) grid = ntiles;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(STREAM_THREADS);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl ? 1 : 0;

  cudaError_t e;
#define IHB_DISPATCH(WT, NI)                                   \
  do {                                                         \
    e = set_smem<WT, NI>(a.epi, smem_bytes);                   \
    if (e != cudaSuccess) return e;                            \
    return launch_epi<WT, NI>(a, cfg);                         \
  } while (0)
  const int nisel = ni <= 1 ? 1 : ni <= 2 ? 2 : ni <= 4 ? 4 : ni <= 8 ? 8 : 16;
  if (a.wtype == IHB_W_FP8) {
    switch (nisel) {
      case 1: IHB_DISPATCH(0, 1);
      case 2: IHB_DISPATCH(0, 2);
      case 4: IHB_DISPATCH(0, 4);
      case 8: IHB_DISPATCH(0, 8);
      default: IHB_DISPATCH(0, 16);
    }
  } else {
    switch (nisel) {
      case 1: IHB_DISPATCH(1, 1);
      case 2: IHB_DISPATCH(1, 2);
      case 4: IHB_DISPATCH(1, 4);
      case 8: IHB_DISPATCH(1, 8);
      default: IHB_DISPATCH(1, 16);
    }
  }
#undef IHB_DISPATCH
}
