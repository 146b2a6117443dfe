// Persistent decode megakernel: ONE cooperative launch runs whole tokens - every layer's QKV GEMV, QK-norm + RoPE +
// KV append + split-KV attention, o_proj, router + top-k, expert gate/up + SwiGLU, expert down, the two
// tensor-parallel all-reduces (partials pushed straight into every GPU's slot buffer through NVSwitch, multimem or
// peer stores) with residual + RMSNorm, the final norm, the vocabulary-sharded head and the cross-rank argmax.
//
// Why: at one token a tensor-parallel layer moves only a few MB per GPU, so a chain of separate kernels is bound
// by launch, prologue and tail latencies, not by bytes. Here a phase hands its result to the next one as tagged
// values the consumer waits on (one grid-wide barrier per layer is left); the residual stream lives in every CTA's
// shared memory (all CTAs add the same partials in the same order, so the copies stay bitwise identical) and the
// activation vector of each GEMV is staged once per CTA in shared memory as pre-scaled fp16.
//
// All CTAs must be resident (cooperative launch, one per SM). Every wait is bounded: on a time-out the error word is
// set, all later waits fall through and the kernel ends normally.
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
  // barrier state: the counters are meaningful in thread 0; epoch (all-reduce rounds so far: slot parity and tag) in
  // every thread; xr counts the rounds on the cross-GPU arrival counter (one per token: the arg-max exchange)
  unsigned base, n_bar, n_prof, epoch, xr;
  // shared memory carve-up
  float* resid;          // [H]
  float* xf;             // [H] fp32 normed hidden state (router input)
  float* xv;             // bf16 weights: fp32 activation vector of the running GEMV
  __half* xh;            // fp8 weights: the activation vector as fp16, pre-scaled by a power of two
  float unscale;         // undoes that pre-scale
  float* red;            // [32] block reductions
  int* sel_e;            // [top_k]
  float* sel_w;          // [top_k]
  int* flags;            // [0] dead, [1] last-arriver flag of the attention merge, [2] routed experts held by this rank,
                         // [3] tag of the vector being produced (GEMV stores and all-reduce pushes)
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
__device__ __forceinline__ void mg_barrier(const IhbMegaArgs& a, MgCtx& c) {
  __syncthreads();
  if (threadIdx.x == 0 && c.flags[0] == 0) {
    c.n_bar++;
    red_release_gpu_add_u32(a.bar + 0, 1u);
    if (!mg_wait(a.bar + 0, c.base + c.n_bar * gridDim.x, a.err)) c.flags[0] = 1;
    if (a.prof != nullptr && blockIdx.x == 0) a.prof[++c.n_prof] = globaltimer_ns();
  }
  __syncthreads();
}

// ---- all-reduce without a barrier: tagged slots ----------------------------------------------------------------------------------
// A partial sum travels as ONE 8-byte store {fp32 value, round tag}: a store of 8 aligned bytes arrives whole, so a
// reader that sees the tag of the round it waits for has the value too, and no fence, arrival counter or barrier is
// needed: the all-reduce costs one one-way trip through NVSwitch. Slots are [parity][rank][H] pairs; the round
// number (never 0, never reused while a slot of that parity can still hold it) is the tag. A slot of round n can be
// overwritten (round n + 2) only by a CTA that has read ALL of round n + 1, which every CTA of every rank pushed
// after it had read round n, so two parities are enough.
__device__ __forceinline__ ulonglong2 ld_relaxed_sys_v2_u64(const unsigned long long* p) {
  ulonglong2 v;
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mg_push(const IhbComm& cm, size_t off, float y, unsigned tag) {
  const unsigned long long v = (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(y);
  unsigned long long* local = reinterpret_cast<unsigned long long*>(cm.slots_local) + off;
  if (cm.nranks == 1) {
    st_relaxed_sys_u64(local, v);
  } else if (cm.slots_mc != nullptr) {
    multimem_st_u64(reinterpret_cast<unsigned long long*>(cm.slots_mc) + off, v);
  } else {
    for (int p = 0; p < cm.nranks; ++p) st_relaxed_sys_u64(reinterpret_cast<unsigned long long*>(cm.slots_peer[p]) + off, v);
  }
}
__device__ __forceinline__ bool mg_tagged(const ulonglong2 (&p)[2], unsigned tag) {
  return static_cast<unsigned>(p[0].x >> 32) == tag && static_cast<unsigned>(p[0].y >> 32) == tag &&
         static_cast<unsigned>(p[1].x >> 32) == tag && static_cast<unsigned>(p[1].y >> 32) == tag;
}
// Re-reads four slots until all carry `tag` (bounded; a set error word ends the wait).
__device__ __forceinline__ bool mg_settle(const unsigned long long* q, ulonglong2 (&p)[2], unsigned tag, unsigned* err) {
  if (mg_tagged(p, tag)) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  for (;;) {
    p[0] = ld_relaxed_sys_v2_u64(q);
    p[1] = ld_relaxed_sys_v2_u64(q + 2);
    if (mg_tagged(p, tag)) return true;
    if ((++spins & 63u) == 0u) {
      if (ld_cg_u(err) != 0u) return false;
      if (globaltimer_ns() - t0 > IHB_PEER_WAIT_NS) { set_error(err, ERR_PEER_BARRIER_TIMEOUT); return false; }
    }
  }
}

// Ask L2 for `bytes` at `p` (all CTAs together, one 128-byte line per thread and round): issued right before the
// wait for the other GPUs' slots, so that this wait brings the next phase's weights on chip.
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

// ---- tagged hand-over between phases on one GPU -----------------------------------------------------------------------------------
// The vectors that one phase writes and the next one reads (QKV, attention output, router logits, expert
// activations) are kept as {fp32 value, tag} pairs too: the consumer waits on the data, no grid barrier separates
// the phases of a layer. Where every CTA consumes, one thread per CTA first polls a sentinel (an element written in
// the producers' last wave), so that idle CTAs do not flood L2 with polls.
__device__ __forceinline__ unsigned long long mg_pack(float v, unsigned tag) {
  return (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(v);
}
__device__ __forceinline__ void st_relaxed_gpu_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// Bounded wait until *p carries `tag`; returns the value (whatever is there after a time-out or a set error word).
__device__ __forceinline__ float mg_ldt(const unsigned long long* p, unsigned tag, unsigned* err) {
  unsigned long long v = ld_relaxed_gpu_u64(p);
  if (static_cast<unsigned>(v >> 32) != tag) {
    const unsigned long long t0 = globaltimer_ns();
    unsigned spins = 0;
    for (;;) {
      v = ld_relaxed_gpu_u64(p);
      if (static_cast<unsigned>(v >> 32) == tag) break;
      if ((++spins & 63u) == 0u) {
        if (ld_cg_u(err) != 0u) break;
        if (globaltimer_ns() - t0 > IHB_LOCAL_WAIT_NS) { set_error(err, ERR_GRID_COUNTER_TIMEOUT); break; }
      }
    }
  }
  return __uint_as_float(static_cast<unsigned>(v));
}
// Second half of a batched tagged read: `raw` was loaded from p earlier (several such loads in flight together); only
// a value whose tag has not arrived yet falls back to the bounded wait.
__device__ __forceinline__ float mg_fix(const unsigned long long* p, unsigned long long raw, unsigned tag, unsigned* err) {
  if (static_cast<unsigned>(raw >> 32) == tag) return __uint_as_float(static_cast<unsigned>(raw));
  return mg_ldt(p, tag, err);
}
// The layer table lives in global memory; its entry for the NEXT layer is copied into shared memory while the current
// layer runs, so that no phase starts with a dependent load of a weight pointer from L2.
__device__ __forceinline__ void mg_fetch_layer(IhbMegaLayer* dst, const IhbMegaLayer* src) {
  static_assert(sizeof(IhbMegaLayer) % 16 == 0, "layer entries are copied in 16-byte pieces");
  if (threadIdx.x < sizeof(IhbMegaLayer) / 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(reinterpret_cast<char*>(dst) + 16 * threadIdx.x)),
                 "l"(reinterpret_cast<const char*>(src) + 16 * threadIdx.x) : "memory");
  asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void mg_fetch_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// End of a phase inside a CTA: shared memory may be reused, CTA 0 records its time.
__device__ __forceinline__ void mg_phase_end(const IhbMegaArgs& a, MgCtx& c) {
  mg_fetch_wait();
  __syncthreads();
  if (a.prof != nullptr && blockIdx.x == 0 && threadIdx.x == 0) a.prof[++c.n_prof] = globaltimer_ns();
}

// mg_stage with U values per thread and round: f(i, v) fills v[u] for index i + u * MG_THREADS (anything past n is
// ignored), so that a source in global memory can have its U loads in flight together.
template <bool FP8, int U, typename F>
__device__ __forceinline__ void mg_stage_batched(MgCtx& c, int n, F f) {
  float m = 0.f;
  for (int i = threadIdx.x; i < n; i += MG_THREADS * U) {
    float v[U];
    f(i, v);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int idx = i + u * MG_THREADS;
      if (idx < n) {
        if (FP8) { m = fmaxf(m, fabsf(v[u])); c.xh[idx] = __float2half_rn(v[u]); }
        else c.xv[idx] = v[u];
      }
    }
  }
  if (FP8) {
    m = block_max(m, c.red);
    c.unscale = 1.f;
    if (m > 8.f) {
      const int e = static_cast<int>(ceilf(log2f(m * 0.125f)));
      const __half hs = __float2half_rn(exp2f(static_cast<float>(-e)));
      c.unscale = exp2f(static_cast<float>(e));
      for (int i = threadIdx.x; i < n; i += MG_THREADS) c.xh[i] = __hmul(c.xh[i], hs);
    }
  }
  __syncthreads();
}

// resid += scale * (the all-reduce round `tag`, summed in rank order so that every rank gets the same bits); returns
// this thread's share of sum(resid^2). ONE thread first polls a sentinel per rank (the slot of the last row, which a
// rank's GEMV writes in its last wave) while the others sleep at a barrier: 75 000 threads polling L2 would slow the
// CTAs that are still streaming weights. Then every thread reads its slots (the loads of up to MG_LLB ranks in
// flight together) and spins only on those that have not landed yet. Kept out of line (scalar arguments only) so
// that its registers do not weigh on the GEMV loops.
constexpr int MG_LLB = 4;
__device__ __noinline__ float mg_reduce_slots(const unsigned long long* base, float* resid, int H, int nr, unsigned tag,
                                              float scale, unsigned* err, bool live) {
  if (threadIdx.x == 0 && live) {
    const unsigned long long t0 = globaltimer_ns();
    unsigned spins = 0;
    bool give_up = false;
    for (int r = 0; r < nr && !give_up; ++r) {
      const unsigned long long* q = base + static_cast<size_t>(r) * H + (H - 2);
      while (static_cast<unsigned>(ld_relaxed_sys_v2_u64(q).y >> 32) != tag) {
        if ((++spins & 63u) == 0u) {
          if (ld_cg_u(err) != 0u) { give_up = true; break; }
          if (globaltimer_ns() - t0 > IHB_PEER_WAIT_NS) { set_error(err, ERR_PEER_BARRIER_TIMEOUT); give_up = true; break; }
        }
      }
    }
  }
  __syncthreads();
  float ss = 0.f;
  bool ok = live;
  for (int i = threadIdx.x * 4; i < H; i += MG_THREADS * 4) {
    float4 v = *reinterpret_cast<float4*>(resid + i);
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r0 = 0; r0 < nr; r0 += MG_LLB) {
      ulonglong2 p[MG_LLB][2];
#pragma unroll
      for (int j = 0; j < MG_LLB; ++j) {
        if (r0 + j < nr) {
          const unsigned long long* q = base + static_cast<size_t>(r0 + j) * H + i;
          p[j][0] = ld_relaxed_sys_v2_u64(q);
          p[j][1] = ld_relaxed_sys_v2_u64(q + 2);
        }
      }
#pragma unroll
      for (int j = 0; j < MG_LLB; ++j) {
        if (r0 + j < nr) {
          if (ok) ok = mg_settle(base + static_cast<size_t>(r0 + j) * H + i, p[j], tag, err);
          sum.x += __uint_as_float(static_cast<unsigned>(p[j][0].x));
          sum.y += __uint_as_float(static_cast<unsigned>(p[j][0].y));
          sum.z += __uint_as_float(static_cast<unsigned>(p[j][1].x));
          sum.w += __uint_as_float(static_cast<unsigned>(p[j][1].y));
        }
      }
    }
    v.x = fmaf(sum.x, scale, v.x); v.y = fmaf(sum.y, scale, v.y); v.z = fmaf(sum.z, scale, v.z); v.w = fmaf(sum.w, scale, v.w);
    *reinterpret_cast<float4*>(resid + i) = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  return ss;
}

// resid (+= the all-reduce round pushed last) -> RMSNorm(gamma) -> xf (fp32) and the staged GEMV input.
template <bool FP8>
__device__ __forceinline__ void mg_residual_norm(const IhbMegaArgs& a, MgCtx& c, bool add_slots, const float* gamma,
                                                 float scale = 1.f) {
  const int H = a.H;
  float ss = 0.f;
  if (add_slots) {
    const unsigned long long* base = reinterpret_cast<const unsigned long long*>(a.comm.slots_local) +
                                     static_cast<size_t>((c.epoch + 1u) & 1u) * a.comm.nranks * H;
    // c.epoch: the round that ended with the last push
    ss = mg_reduce_slots(base, c.resid, H, a.comm.nranks, c.epoch, scale, a.err, c.flags[0] == 0);
  } else {
    for (int i = threadIdx.x * 4; i < H; i += MG_THREADS * 4) {
      const float4 v = *reinterpret_cast<float4*>(c.resid + i);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  }
  const float tot = block_sum(ss, c.red);
  if (add_slots && a.prof != nullptr && blockIdx.x == 0 && threadIdx.x == 0) a.prof[++c.n_prof] = globaltimer_ns();
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
// loop is instantiated once per (R, U), force-inlined: the whole kernel has to stay small for the instruction cache.
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
  float* out;                    // STORE: {value, tag} pairs (the tag waits in c.flags[3]); ARGMAX: optional logits
  size_t off;                    // PUSH: slot offset of this rank (the round's tag waits in c.flags[3])
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
          st_relaxed_gpu_u64(reinterpret_cast<unsigned long long*>(sink.out) + i,
                             mg_pack(v, static_cast<unsigned>(*reinterpret_cast<volatile int*>(c.flags + 3))));
        } else if (sink.kind == MG_PUSH) {
          mg_push(a.comm, sink.off + i, v, static_cast<unsigned>(*reinterpret_cast<volatile int*>(c.flags + 3)));
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
