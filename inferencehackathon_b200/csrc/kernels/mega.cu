// Persistent decode megakernel: ONE cooperative launch runs whole tokens - every layer's QKV GEMV, QK-norm + RoPE +
// KV append + split-KV attention, o_proj, router + top-k, expert gate/up + SwiGLU, expert down, the two
// tensor-parallel all-reduces (partials pushed straight into every GPU's slot buffer through NVSwitch, multimem or
// peer stores) with residual + RMSNorm, the final norm, the vocabulary-sharded head and the cross-rank argmax.
//
// Why: at one token a tensor-parallel layer moves only a few MB per GPU, so a chain of separate kernels is bound
// by launch, prologue and tail latencies, not by bytes. Here the phases of a layer are separated by a grid-wide
// barrier (one atomic arrival per CTA + a spin on one counter); the residual stream lives in every CTA's shared
// memory (all CTAs add the same partials in the same order, so the copies stay bitwise identical) and the
// activation vector of each GEMV is staged once per CTA in shared memory as pre-scaled fp16.
//
// All CTAs must be resident (cooperative launch, one per SM). Every wait is bounded: on a time-out the error word is
// set, all later barriers fall through and the kernel ends normally.
//
// The reference's persistent kernel (kernels/megakernel_decode.cu:575-649) pays ~16 cooperative grid syncs and
// NVSHMEM barriers per layer and measured 9-11x slower than its multi-kernel path (docs/path-to-1000.md:32-34).
#include <algorithm>
#include "common.cuh"
#include "tails.cuh"

namespace ihb {

constexpr int MG_THREADS = 512;
constexpr int MG_WARPS = 16;
constexpr int MG_HD = 128;
constexpr int MG_GQ = 8;                 // query heads per attention work item
constexpr int MG_REC = MG_HD + 4;        // attention partial record: acc[128], m, l, 2 pad (16-byte multiple)

constexpr int MG_NPB = 4;                // blocks of 32 positions per CTA round
constexpr int MG_WPB = MG_WARPS / MG_NPB;      // warps sharing a block; each takes MG_HW of the 8 query heads
constexpr int MG_HW = MG_GQ / MG_WPB;
constexpr int MG_ABLK = MG_NPB * 32;           // positions per CTA round

struct MgAttnSmem {
  float q[MG_GQ][MG_HD];
  float p[MG_WARPS][MG_HW][32];
  float m[MG_WARPS][MG_HW], l[MG_WARPS][MG_HW];
  float acc[MG_WARPS][MG_HW][MG_HD];
  __nv_bfloat16 knew[MG_HD], vnew[MG_HD];
  // K rows of the block a warp pair works on: loaded row-contiguous (coalesced), read one row per lane; the 16-byte
  // pad per row spreads the rows of a quarter warp over all banks
  __align__(16) __nv_bfloat16 kst[MG_NPB][32][MG_HD + 8];
};

struct MgCtx {
  // barrier state: the counters are meaningful in thread 0; epoch (cross-GPU rounds so far) in every thread
  unsigned base, n_bar, n_prof, epoch;
  // shared memory carve-up
  float* resid;          // [H]
  float* xf;             // [H] fp32 normed hidden state (router input)
  float* xv;             // bf16 weights: fp32 activation vector of the running GEMV
  __half* xh;            // fp8 weights: the activation vector as fp16, pre-scaled by a power of two
  float unscale;         // undoes that pre-scale
  float* red;            // [32] block reductions
  int* sel_e;            // [top_k]
  float* sel_w;          // [top_k]
  int* flags;            // [0] dead, [1] last-arriver flag of the attention merge, [2] routed experts held by this rank
  MgAttnSmem* attn;
};

__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Bounded spin (thread 0) until *ctr - target >= 0. A set error word ends every wait at once.
__device__ __forceinline__ bool mg_wait(const unsigned* ctr, unsigned target, unsigned* err) {
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (static_cast<int>(ld_acquire_gpu_u32(ctr) - target) < 0) {
    if ((++spins & 127u) == 0u) {
      if (ld_cg_u(err) != 0u) return false;
      if (globaltimer_ns() - t0 > IHB_LOCAL_WAIT_NS) { set_error(err, ERR_GRID_COUNTER_TIMEOUT); return false; }
    }
  }
  return true;
}

__device__ __forceinline__ void red_release_gpu_add_u32(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded spin on this GPU's cross-GPU arrival counter (system-scope acquire).
__device__ __forceinline__ bool mg_wait_sys(const unsigned* flag, unsigned target, unsigned* err) {
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (static_cast<int>(ld_acquire_sys_u32(flag) - target) < 0) {
    if ((++spins & 63u) == 0u) {
      if (ld_cg_u(err) != 0u) return false;
      if (globaltimer_ns() - t0 > IHB_PEER_WAIT_NS) { set_error(err, ERR_PEER_BARRIER_TIMEOUT); return false; }
    }
  }
  return true;
}

// `count` arrivals of this rank on every GPU's counter (one multicast reduction, or one per peer).
__device__ __forceinline__ void mg_arrive_all(const IhbComm& cm, unsigned count) {
  if (cm.flag_mc != nullptr) {
    multimem_red_release_sys_add_u32(cm.flag_mc, count);
  } else {
    for (int r = 0; r < cm.nranks; ++r) red_release_sys_add_u32(cm.flag_peer[r], count);
  }
}

// Grid-wide barrier: one fire-and-forget release-add per CTA, then a spin on the same counter.
// cross = true (several GPUs): every CTA of every rank arrives directly on every GPU's counter - its partials were
// pushed before, the release orders them - and waits until all ranks x CTAs of this round are in: one NVLink round
// trip, no local hop before or after it. The counter advances by nranks * gridDim.x per cross-GPU round.
__device__ __forceinline__ void mg_barrier(const IhbMegaArgs& a, MgCtx& c, bool cross) {
  __syncthreads();
  if (threadIdx.x == 0 && c.flags[0] == 0) {
    bool ok = true;
    if (cross && a.comm.nranks > 1) {
      // release at system scope: the CTA's pushes (ordered before thread 0 by the barrier above) become visible to
      // whoever acquires the counter; an acq_rel fence is enough here and cheaper than the sequentially consistent
      // one __threadfence_system() issues
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      mg_arrive_all(a.comm, 1u);
      ok = mg_wait_sys(a.comm.flag_local, (c.epoch + 1u) * static_cast<unsigned>(a.comm.nranks) * gridDim.x, a.err);
    } else {
      c.n_bar++;
      red_release_gpu_add_u32(a.bar + 0, 1u);
      ok = mg_wait(a.bar + 0, c.base + c.n_bar * gridDim.x, a.err);
    }
    if (!ok) c.flags[0] = 1;
    if (a.prof != nullptr && blockIdx.x == 0) a.prof[++c.n_prof] = globaltimer_ns();
  }
  if (cross) c.epoch++;          // every thread keeps the count of cross-GPU rounds (it selects the slot parity)
  __syncthreads();
}

// Ask L2 for `bytes` at `p` (all CTAs together, one 128-byte line per thread and round): issued right before a
// cross-GPU barrier, so that the wait for the other GPUs brings the next phase's weights on chip.
__device__ __forceinline__ void mg_prefetch_l2(const void* p, size_t bytes) {
  const char* base = reinterpret_cast<const char*>(p);
  const size_t step = static_cast<size_t>(gridDim.x) * MG_THREADS * 128;
  for (size_t off = (static_cast<size_t>(blockIdx.x) * MG_THREADS + threadIdx.x) * 128; off < bytes; off += step)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < MG_WARPS; ++w) t += red[w];
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = red[0];
#pragma unroll
  for (int w = 1; w < MG_WARPS; ++w) t = fmaxf(t, red[w]);
  return t;
}

// Stages the n values f(i) (one global read each at most) as the activation vector of the next GEMV. fp8 weights:
// fp16 in shared memory, scaled by a power of two so that max|x| <= 8, which bounds the fp16 accumulation chains of
// dot16_e4m3 (the values are stored at once and re-scaled in place only when needed: a power-of-two factor, so no
// second rounding); bf16 weights: fp32.
template <bool FP8, typename F>
__device__ __forceinline__ void mg_stage(MgCtx& c, int n, F f) {
  if (FP8) {
    float m = 0.f;
    for (int i = threadIdx.x; i < n; i += MG_THREADS) {
      const float v = f(i);
      m = fmaxf(m, fabsf(v));
      c.xh[i] = __float2half_rn(v);
    }
    m = block_max(m, c.red);
    c.unscale = 1.f;
    if (m > 8.f) {
      const int e = static_cast<int>(ceilf(log2f(m * 0.125f)));
      const __half hs = __float2half_rn(exp2f(static_cast<float>(-e)));
      c.unscale = exp2f(static_cast<float>(e));
      for (int i = threadIdx.x; i < n; i += MG_THREADS) c.xh[i] = __hmul(c.xh[i], hs);
    }
  } else {
    for (int i = threadIdx.x; i < n; i += MG_THREADS) c.xv[i] = f(i);
  }
  __syncthreads();
}

// resid (+= the all-reduce slots of `parity`, in rank order) -> RMSNorm(gamma) -> xf (fp32) and the staged GEMV input.
template <bool FP8>
__device__ __forceinline__ void mg_residual_norm(const IhbMegaArgs& a, MgCtx& c, bool add_slots, int parity,
                                                 const float* gamma, float scale = 1.f) {
  const int H = a.H;
  const int nr = a.comm.nranks;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < H; i += MG_THREADS * 4) {
    float4 v = *reinterpret_cast<float4*>(c.resid + i);
    if (add_slots) {
      const float* sl = a.comm.slots_local + static_cast<size_t>(parity) * nr * H + i;
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < nr; ++r) {
        const float4 p = ld_cg_f4(reinterpret_cast<const float4*>(sl + static_cast<size_t>(r) * H));
        sum.x += p.x; sum.y += p.y; sum.z += p.z; sum.w += p.w;
      }
      v.x = fmaf(sum.x, scale, v.x); v.y = fmaf(sum.y, scale, v.y); v.z = fmaf(sum.z, scale, v.z); v.w = fmaf(sum.w, scale, v.w);
      *reinterpret_cast<float4*>(c.resid + i) = v;
    }
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  const float tot = block_sum(ss, c.red);
  const float rinv = rsqrtf(tot / static_cast<float>(H) + a.eps);
  for (int i = threadIdx.x * 4; i < H; i += MG_THREADS * 4) {
    const float4 v = *reinterpret_cast<float4*>(c.resid + i);
    const float4 g = *reinterpret_cast<const float4*>(gamma + i);
    *reinterpret_cast<float4*>(c.xf + i) = make_float4(v.x * rinv * g.x, v.y * rinv * g.y, v.z * rinv * g.z, v.w * rinv * g.w);
  }
  __syncthreads();
  const float* xf = c.xf;
  mg_stage<FP8>(c, H, [xf](int i) { return xf[i]; });
}

// ---- GEMV building block ----------------------------------------------------------------------------------------------------
// A "virtual row" is a list of 16-byte weight chunks; chunk c multiplies activation elements [EPC c, EPC c + EPC)
// (EPC = 16 for e4m3, 8 for bf16). A warp takes groups of R consecutive rows and keeps R x U independent 16-byte loads
// in flight per lane. ONE plan type covers the three matrix layouts and one sink type the three result uses, so the
// loop is instantiated once per (R, U) and not inlined: the whole kernel has to stay small for the instruction cache.
//   PLAIN  rows x rowbytes
//   EXPERT gate/up of the routed experts: virtual row v = slot * rpe + jj (rpe = 2 I rows per expert)
//   DOWN   output rows over all routing slots: chunk c -> (expert of slot c / nch1, chunk c % nch1 of its row)
//          through a table of offsets in shared memory (the same for every row, built once per layer)
enum { MG_PLAIN = 0, MG_EXPERT = 1, MG_DOWN = 2 };
struct MgPlan {
  int kind;
  const uint8_t* W; const float* sc;
  int rows, nch, rowbytes, rb, kbs, nkb, rpe, nrb;
  const int* sel_e;
  const uint2* tab;
};
struct RowBase { const uint8_t* w; const float* s; };

__device__ __forceinline__ RowBase mg_row(const MgPlan& pl, int v) {
  if (pl.kind == MG_EXPERT) {
    const int slot = v / pl.rpe, jj = v - slot * pl.rpe;
    const size_t e = static_cast<size_t>(pl.sel_e[slot]);
    return RowBase{pl.W + (e * pl.rpe + jj) * pl.rowbytes, pl.sc + (e * pl.nrb + jj / pl.rb) * pl.nkb};
  }
  return RowBase{pl.W + static_cast<size_t>(v) * pl.rowbytes, pl.sc + static_cast<size_t>(v / pl.rb) * pl.nkb};
}

enum { MG_STORE = 0, MG_PUSH = 1, MG_ARGMAX = 2 };
struct MgSink {
  int kind;
  float* out;                    // STORE: out[i]; ARGMAX: optional logits
  size_t off;                    // PUSH: slot offset of this rank
  unsigned long long best;       // ARGMAX: packed running maximum (lane 0 of each warp)
};

template <bool FP8>
__device__ __forceinline__ float mg_chunk_dot(uint4 w, const __half* xh, const float* xv, int cch) {
  if (FP8) {
    const uint4* x = reinterpret_cast<const uint4*>(xh + 16 * cch);
    return dot16_e4m3(w, x[0], x[1]);
  } else {
    const float4* x = reinterpret_cast<const float4*>(xv + 8 * cch);
    return dot8_bf16(w, x[0], x[1]);
  }
}

template <bool FP8, int R, int U>
__device__ __forceinline__ void mg_gemv(const IhbMegaArgs& a, const MgCtx& c, const MgPlan& plan, MgSink& sink) {
  const int lane = threadIdx.x & 31;
  const int first = blockIdx.x * MG_WARPS + (threadIdx.x >> 5);     // the warps of a CTA read one contiguous run
  const int stride = gridDim.x * MG_WARPS;
  const int n = plan.rows, nch = plan.nch, kbs = plan.kbs;
  const __half* xh = c.xh;
  const float* xv = c.xv;
  const float unscale = FP8 ? c.unscale : 1.f;
  const bool down = plan.kind == MG_DOWN;
  for (int i0 = first * R; i0 < n; i0 += stride * R) {
    RowBase b[R];
    float acc[R];
#pragma unroll
    for (int j = 0; j < R; ++j) {
      b[j] = mg_row(plan, min(i0 + j, n - 1));
      acc[j] = 0.f;
    }
    for (int cb = 0; cb < nch; cb += 32 * U) {
      uint4 w[R][U];
      float s[R][U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int cch = cb + lane + 32 * u;
        const bool valid = cch < nch;
        unsigned wo = 0, so = 0;
        if (valid) {
          if (down) { const uint2 t = plan.tab[cch]; wo = t.x; so = t.y; }
          else { wo = 16u * cch; so = cch >> kbs; }
        }
#pragma unroll
        for (int j = 0; j < R; ++j) {
          w[j][u] = valid ? ldg_stream(b[j].w + wo) : make_uint4(0u, 0u, 0u, 0u);
          s[j][u] = (FP8 && valid) ? __ldg(b[j].s + so) : (valid ? 1.f : 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int cch = min(cb + lane + 32 * u, nch - 1);
#pragma unroll
        for (int j = 0; j < R; ++j) acc[j] = fmaf(s[j][u], mg_chunk_dot<FP8>(w[j][u], xh, xv, cch), acc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const float v = warp_sum(acc[j]) * unscale;
      const int i = i0 + j;
      if (lane == 0 && i < n) {
        if (sink.kind == MG_STORE) {
          sink.out[i] = v;
        } else if (sink.kind == MG_PUSH) {
          push_partial(a.comm, sink.off + i, v);
        } else {
          const unsigned long long pk = pack_max(v, static_cast<unsigned>(i));
          sink.best = pk > sink.best ? pk : sink.best;
          if (sink.out != nullptr) sink.out[i] = v;
        }
      }
    }
  }
}

// Picks the (rows, rounds) shape by the number of chunk rounds a row needs and by how many rows a warp gets.
template <bool FP8>
__device__ __forceinline__ void mg_gemv_auto(const IhbMegaArgs& a, const MgCtx& c, const MgPlan& plan, MgSink& sink) {
  const int W = gridDim.x * MG_WARPS;
  if (plan.kind == MG_DOWN && plan.nch > 128 && plan.rows >= 3 * W) mg_gemv<FP8, 4, 4>(a, c, plan, sink);   // longer runs per expert
  else if (plan.nch > 128 && plan.rows >= 2 * W) mg_gemv<FP8, 2, 8>(a, c, plan, sink);
  else if (plan.nch > 128) mg_gemv<FP8, 1, 8>(a, c, plan, sink);
  else if (plan.nch > 64) mg_gemv<FP8, 2, 4>(a, c, plan, sink);
  else mg_gemv<FP8, 4, 2>(a, c, plan, sink);
}

__device__ __forceinline__ MgPlan mg_plan(int kind, const IhbMat& m, int rows, int nch, int rowbytes, const int* sel_e,
                                          int rpe, const uint2* tab) {
  MgPlan pl;
  pl.kind = kind; pl.W = m.W; pl.sc = m.wscale; pl.rows = rows; pl.nch = nch; pl.rowbytes = rowbytes;
  pl.rb = m.rb > 0 ? m.rb : (1 << 30); pl.kbs = m.kb_shift; pl.nkb = m.nkb;
  pl.rpe = rpe; pl.sel_e = sel_e; pl.tab = tab;
  pl.nrb = m.rb > 0 ? ((kind == MG_EXPERT ? rpe : rows) + m.rb - 1) / m.rb : 0;
  return pl;
}

#include "mega_phases.inc"

}  // namespace ihb

#include "mega_host.inc"
