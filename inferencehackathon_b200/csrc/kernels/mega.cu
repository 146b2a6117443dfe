// Persistent decode megakernel: ONE cooperative launch runs whole tokens - every layer's QKV GEMV, QK-norm + RoPE +
// KV append + split-KV attention, o_proj, router + top-k, expert gate/up + SwiGLU, expert down, the two
// tensor-parallel all-reduces (partials added straight into every GPU's slot buffer through NVSwitch, multimem.red or
// peer reds) with residual + RMSNorm, the final norm, the vocabulary-sharded head and the cross-rank argmax.
//
// Why: at one token a tensor-parallel layer moves only a few MB per GPU, so a chain of separate kernels is bound
// by launch, prologue and tail latencies, not by bytes. Here a phase hands its result to the next one as tagged
// values the consumer waits on; the two all-reduces of a layer are counted fixed-point accumulations (every rank adds
// its partial into every GPU's slot with one multimem.red / peer red, the reader waits for the contribution count);
// the residual stream lives in every CTA's shared memory (all CTAs read the same integer sums, so the copies stay
// bitwise identical on every CTA of every GPU) and the activation vector of each GEMV is staged once per CTA in
// shared memory as pre-scaled fp16.
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

// Attention work item of the consumer-merge mode: one block of MG_ABLK positions whose K / V rows were copied into
// shared memory (cp.async) while the QKV projection was still running.
struct MgAttn2 {
  // rows padded by 16 bytes: the 32-bit fragment loads of a quarter warp and the 16-byte rows of an ldmatrix then
  // cover all banks
  __align__(16) __nv_bfloat16 qh[MG_GQ][MG_HD + 8];     // scaled q, split into a bf16 head and a bf16 remainder
  __align__(16) __nv_bfloat16 ql[MG_GQ][MG_HD + 8];
  __align__(16) __nv_bfloat16 ph[MG_GQ][MG_ABLK + 8];   // probabilities of the block, split the same way
  __align__(16) __nv_bfloat16 pl[MG_GQ][MG_ABLK + 8];
  __align__(16) float sc[MG_GQ][MG_ABLK];               // scores (log2 domain)
  float hm[MG_GQ], hl[MG_GQ];                           // per head: maximum, sum of probabilities
  __align__(16) __nv_bfloat16 knew[MG_HD];
  __align__(16) __nv_bfloat16 vnew[MG_HD];
  __align__(16) __nv_bfloat16 kst[MG_ABLK][MG_HD + 8];
  __align__(16) __nv_bfloat16 vst[MG_ABLK][MG_HD + 8];
};
constexpr int MG_RSPL = 16;              // splits per head in the record buffer of the consumer-merge mode
constexpr int MG_MERGE_MAX = 256;        // (head, split) records a consumer CTA is willing to merge
constexpr int MG_RECW = MG_HD / 2 + 2;   // 8-byte words per record: 64 {half2, tag} pairs, {m, tag}, {l, tag}
struct MgMerge { float m[MG_MERGE_MAX], l[MG_MERGE_MAX]; };
constexpr size_t MG_ATTN_SMEM = sizeof(MgAttn2) > sizeof(MgAttnSmem) ? sizeof(MgAttn2) : sizeof(MgAttnSmem);

// The code of this kernel runs once per layer, so whatever is inlined at several places is fetched again from L2 at
// every one of them (the kernel is far larger than the instruction caches): the GEMV with all its shapes and the
// residual + norm step are therefore compiled ONCE, out of line. Their arguments travel through this block of
// shared memory (a structure passed by reference would live in local memory and slow the streaming loops down).
struct MgPlan {
  int kind;
  const uint8_t* W; const float* sc;
  int rows, nch, rowbytes, rb, kbs, nkb, rpe, nrb;
  const int* sel_e;
  const uint2* tab;
};
struct MgSink {
  int kind;
  float* out;                    // STORE: {value, tag} pairs (the tag waits in flags[3]); ARGMAX: optional logits
  size_t off;                    // PUSH: slot offset of the round's parity
};
struct MgShm {
  float red[32];                 // block reductions
  int sel_e[IHB_MAX_TOPK];       // routed experts this rank holds (local ids, slot order) and their weights
  float sel_w[IHB_MAX_TOPK];
  int topi[IHB_MAX_TOPK];
  float topl[IHB_MAX_TOPK];
  unsigned keys[256];
  float lgs[256];
  int flags[4];                  // [0] dead, [1] last-arriver flag of the attention merge, [2] routed experts held by this
                                 // rank, [3] tag of the vector being produced (GEMV stores)
  unsigned long long best[MG_WARPS];
  MgPlan plan;                   // arguments of the running GEMV: written by thread 0 before a CTA barrier
  MgSink sink;
  __align__(16) IhbMegaLayer ly[2];
};
// Dynamic shared memory: [MgShm][resid H fp32][xf H fp32][activation vector][attention scratch]. Every function derives
// its pointers from this array itself, so that the compiler knows they are shared-memory addresses (a pointer read
// from memory would be a generic one, and the GEMV's activation reads would turn into generic loads).
extern __shared__ __align__(16) uint8_t mg_smem[];
constexpr size_t MG_SHM_BYTES = (sizeof(MgShm) + 15) & ~size_t(15);
__device__ __forceinline__ MgShm& mg_shm() { return *reinterpret_cast<MgShm*>(mg_smem); }

struct MgCtx {
  // barrier state: the counters are meaningful in thread 0; epoch (all-reduce rounds so far: slot parity and tag) in
  // every thread; xr counts the rounds on the cross-GPU arrival counter (one per token: the arg-max exchange)
  unsigned base, n_bar, epoch, xr;
  unsigned clr_lo;       // first all-reduce round whose slots have not been cleared yet
  unsigned ar_n;         // contributions that complete an all-reduce slot
  int layer;             // layer being computed (detail stamps of the profile)
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
                         // [3] tag of the vector being produced (GEMV stores)
  MgAttnSmem* attn;
  MgAttn2* attn2;        // same bytes as attn
};
template <bool FP8>
__device__ __forceinline__ void mg_ctx_pointers(const IhbMegaArgs& a, MgCtx& c) {
  MgShm& sh = mg_shm();
  const int maxk = max(max(a.H, a.nq * MG_HD), a.top_k * a.I);
  uint8_t* p = mg_smem + MG_SHM_BYTES;
  c.resid = reinterpret_cast<float*>(p);            p += sizeof(float) * a.H;
  c.xf = reinterpret_cast<float*>(p);               p += sizeof(float) * a.H;
  c.xv = reinterpret_cast<float*>(p);               p += FP8 ? 0 : sizeof(float) * maxk;
  c.xh = reinterpret_cast<__half*>(p);              p += FP8 ? sizeof(__half) * maxk : 0;
  p = mg_smem + ((static_cast<size_t>(p - mg_smem) + 15) & ~size_t(15));
  c.attn = reinterpret_cast<MgAttnSmem*>(p);
  c.attn2 = reinterpret_cast<MgAttn2*>(p);
  c.red = sh.red; c.sel_e = sh.sel_e; c.sel_w = sh.sel_w; c.flags = sh.flags;
}

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

// Per-phase time stamps (profiling runs only): CTA 0's own clock at `idx`, and the latest clock of any CTA at
// prof_n + idx, so that the table shows both when CTA 0 and when the slowest CTA left a phase.
__device__ __forceinline__ void mg_stamp(const IhbMegaArgs& a, int idx) {
  if (a.prof != nullptr && threadIdx.x == 0) {
    const unsigned long long t = globaltimer_ns();
    if (blockIdx.x == 0) a.prof[idx] = t;
    atomicMax(a.prof + a.prof_n + idx, t);
  }
}

// Detail stamps (builds with -DIHB_MEGA_DETAIL and profiling runs only: they perturb the code layout): thread 0 of the
// LAST CTA, which runs the first attention work item, records up to 32 points per layer at [2 prof_n + 32 layer + k].
__device__ __forceinline__ void mg_detail(const IhbMegaArgs& a, const MgCtx& c, int k) {
#ifdef IHB_MEGA_DETAIL
  if (a.prof != nullptr && threadIdx.x == 0 && blockIdx.x == gridDim.x - 1)
    a.prof[2 * a.prof_n + 32 * c.layer + k] = globaltimer_ns();
#endif
}

// Grid-wide barrier: one fire-and-forget release-add per CTA, then a spin on the same counter. The two halves can be
// issued apart: every CTA arrives as soon as its own work is published and waits only where it needs the others.
__device__ __forceinline__ void mg_barrier_arrive(const IhbMegaArgs& a, MgCtx& c) {
  if (threadIdx.x == 0 && c.flags[0] == 0) {
    c.n_bar++;
    red_release_gpu_add_u32(a.bar + 0, 1u);
  }
}
__device__ __forceinline__ void mg_barrier_wait(const IhbMegaArgs& a, MgCtx& c) {
  if (threadIdx.x == 0 && c.flags[0] == 0) {
    if (!mg_wait(a.bar + 0, c.base + c.n_bar * gridDim.x, a.err)) c.flags[0] = 1;
  }
  __syncthreads();
}
__device__ __forceinline__ void mg_barrier(const IhbMegaArgs& a, MgCtx& c) {
  __syncthreads();
  mg_barrier_arrive(a, c);
  mg_barrier_wait(a, c);
}

// ---- all-reduce without a barrier: counted fixed-point accumulation -----------------------------------------------------------------
// A slot is one 64-bit word per hidden channel: the top 8 bits count contributions, the low 56 bits hold the sum of
// the ranks' partials as biased fixed point (28 fraction bits). A rank contributes with ONE 64-bit add on every GPU's
// copy of the slot (multimem.red through NVSwitch, or one red per peer); the reader polls until the count equals the
// number of ranks and then owns the sum: one one-way trip, no fence, no arrival counter, no barrier, and the reader
// moves 8 bytes per channel whatever the number of ranks. Integer addition is associative, so every GPU decodes the
// same bits in whatever order the adds landed - the ranks stay in lock step without a fixed summation order.
// Slots are [MG_NPAR round parities][H]; a round's slots are cleared by the local CTAs after the grid barrier that
// follows their last reader and are used again MG_NPAR rounds later.
constexpr int MG_NPAR = 8;
constexpr unsigned long long MG_ONE = 1ull << 56;
constexpr long long MG_BIAS = 1ll << 51, MG_QMAX = 1ll << 50;
constexpr float MG_FIX = 268435456.f;    // 2^28: |partial| < 2^22, resolution 3.7e-9

__device__ __forceinline__ unsigned long long mg_encode(float v) {
  long long q = __float2ll_rn(v * MG_FIX);
  q = q > MG_QMAX ? MG_QMAX : (q < -MG_QMAX ? -MG_QMAX : q);
  return MG_ONE + static_cast<unsigned long long>(q + MG_BIAS);
}
__device__ __forceinline__ float mg_decode(unsigned long long w, unsigned n) {
  const long long s = static_cast<long long>(w & (MG_ONE - 1ull)) - static_cast<long long>(n) * MG_BIAS;
  return __ll2float_rn(s) * (1.f / MG_FIX);
}
__device__ __forceinline__ void red_relaxed_sys_add_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void multimem_red_add_u64(unsigned long long* mc, unsigned long long v) {
  asm volatile("multimem.red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(mc), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ ulonglong2 ld_relaxed_sys_v2_u64(const unsigned long long* p) {
  ulonglong2 v;
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
  return v;
}
// This rank's partial y of channel `off` (slot parity included) goes to every GPU. With one rank and
// ar_loopback = k > 1 the word receives k adds (the value once, zero k - 1 times): the traffic of k ranks on one
// GPU, for profiling without peers.
__device__ __forceinline__ void mg_push(const IhbMegaArgs& a, size_t off, float y) {
  const IhbComm& cm = a.comm;
  const unsigned long long w = mg_encode(y);
  if (cm.nranks == 1) {
    unsigned long long* local = reinterpret_cast<unsigned long long*>(cm.slots_local) + off;
    if (a.ar_loopback <= 1) {
      st_relaxed_sys_u64(local, w);
    } else {
      red_relaxed_sys_add_u64(local, w);
      for (int k = 1; k < a.ar_loopback; ++k) red_relaxed_sys_add_u64(local, MG_ONE + static_cast<unsigned long long>(MG_BIAS));
    }
  } else if (cm.slots_mc != nullptr) {
    multimem_red_add_u64(reinterpret_cast<unsigned long long*>(cm.slots_mc) + off, w);
  } else {
    for (int p = 0; p < cm.nranks; ++p) red_relaxed_sys_add_u64(reinterpret_cast<unsigned long long*>(cm.slots_peer[p]) + off, w);
  }
}
__device__ __forceinline__ bool mg_counted(const ulonglong2 (&p)[2], unsigned n) {
  return static_cast<unsigned>(p[0].x >> 56) == n && static_cast<unsigned>(p[0].y >> 56) == n &&
         static_cast<unsigned>(p[1].x >> 56) == n && static_cast<unsigned>(p[1].y >> 56) == n;
}
// Slow path of a slot read, out of line (the spin loops would otherwise be copied into every unrolled read): re-reads
// four slots until all hold n contributions (bounded; a set error word ends the wait).
__device__ __noinline__ bool mg_wait_counted(const unsigned long long* q, unsigned n, unsigned* err) {
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  for (;;) {
    ulonglong2 p[2];
    p[0] = ld_relaxed_sys_v2_u64(q);
    p[1] = ld_relaxed_sys_v2_u64(q + 2);
    if (mg_counted(p, n)) return true;
    if ((++spins & 63u) == 0u) {
      if (ld_cg_u(err) != 0u) return false;
      if (globaltimer_ns() - t0 > IHB_PEER_WAIT_NS) { set_error(err, ERR_PEER_BARRIER_TIMEOUT); return false; }
    }
  }
}
// The local CTAs clear the slots of the rounds [c.clr_lo, c.epoch): called after a grid barrier that every CTA passed
// after reading those rounds. The next adds into these words come MG_NPAR rounds later.
__device__ __forceinline__ void mg_clear_read_rounds(const IhbMegaArgs& a, MgCtx& c) {
  unsigned long long* slots = reinterpret_cast<unsigned long long*>(a.comm.slots_local);
  for (unsigned r = c.clr_lo; r != c.epoch; ++r) {
    unsigned long long* s = slots + static_cast<size_t>(r & (MG_NPAR - 1)) * a.H;
    for (int i = blockIdx.x * MG_THREADS + threadIdx.x; i < a.H; i += gridDim.x * MG_THREADS) st_relaxed_sys_u64(s + i, 0ull);
  }
  c.clr_lo = c.epoch;
}

// Ask L2 for `bytes` at `p` (all CTAs together, one 128-byte line per thread and round): issued right before a
// wait, so that the wait brings the next phase's weights on chip.
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
// Sum of s and maximum of m over the CTA with one pair of barriers.
__device__ __forceinline__ float2 block_sum_max(float s, float m, float* red) {
  s = warp_sum(s);
  m = warp_max(m);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = s; red[MG_WARPS + (threadIdx.x >> 5)] = m; }
  __syncthreads();
  float ts = 0.f, tm = 0.f;
#pragma unroll
  for (int w = 0; w < MG_WARPS; ++w) { ts += red[w]; tm = fmaxf(tm, red[MG_WARPS + w]); }
  return make_float2(ts, tm);
}

// Staging of the activation vector of the next GEMV. fp8 weights: fp16 in shared memory, scaled by a power of two so
// that max|x| <= 8, which bounds the fp16 accumulation chains of dot16_e4m3 (the values are stored at once and
// re-scaled in place only when needed: a power-of-two factor, so no second rounding); bf16 weights: fp32.
template <bool FP8>
__device__ __forceinline__ void mg_stage_put(MgCtx& c, int idx, float v, float& m) {
  if (FP8) { m = fmaxf(m, fabsf(v)); c.xh[idx] = __float2half_rn(v); }
  else c.xv[idx] = v;
}
template <bool FP8>
__device__ __forceinline__ void mg_stage_finish(MgCtx& c, int n, float m) {
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

// ---- tagged hand-over between phases on one GPU -----------------------------------------------------------------------------------
// The vectors that one phase writes and the next one reads (QKV, attention records, router logits, expert
// activations) are {fp32 value, tag} pairs: one aligned 8-byte store arrives whole, so a reader that sees the tag of
// the round it waits for has the value. The consumer waits on the data, no grid barrier separates the phases. Where
// every CTA consumes, one thread or warp per CTA first polls a sentinel (an element written in the producers' last
// wave), so that idle CTAs do not flood L2 with polls. Every CTA pushes rows in every all-reduce round (the host
// keeps the grid <= H / 4), so a CTA that has read round r knows that every CTA of every GPU has left everything
// that precedes its push of round r: that orders the reuse of these single-buffered vectors one layer later.
__device__ __forceinline__ unsigned mg_tag(unsigned epoch) { return (epoch & 0x3fffffffu) + 1u; }      // never 0
__device__ __forceinline__ unsigned long long mg_pack(float v, unsigned tag) {
  return (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(v);
}
__device__ __forceinline__ unsigned long long mg_pack_u(unsigned v, unsigned tag) {
  return (static_cast<unsigned long long>(tag) << 32) | v;
}
__device__ __forceinline__ void st_relaxed_gpu_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_gpu_v2_u64(unsigned long long* p, unsigned long long x, unsigned long long y) {
  asm volatile("st.relaxed.gpu.global.v2.b64 [%0], {%1, %2};" ::"l"(p), "l"(x), "l"(y) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// Bounded wait until *p carries `tag`; returns the 32-bit payload (whatever is there after a time-out or a set error
// word). Out of line: it is the slow path of every tagged read.
__device__ __noinline__ unsigned mg_wait_tag(const unsigned long long* p, unsigned tag, unsigned* err) {
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  unsigned long long v;
  for (;;) {
    v = ld_relaxed_gpu_u64(p);
    if (static_cast<unsigned>(v >> 32) == tag) break;
    if ((++spins & 63u) == 0u) {
      if (ld_cg_u(err) != 0u) break;
      if (globaltimer_ns() - t0 > IHB_LOCAL_WAIT_NS) { set_error(err, ERR_GRID_COUNTER_TIMEOUT); break; }
    }
  }
  return static_cast<unsigned>(v);
}
__device__ __forceinline__ unsigned mg_ldt_u(const unsigned long long* p, unsigned tag, unsigned* err) {
  const unsigned long long v = ld_relaxed_gpu_u64(p);
  if (static_cast<unsigned>(v >> 32) == tag) return static_cast<unsigned>(v);
  return mg_wait_tag(p, tag, err);
}
__device__ __forceinline__ float mg_ldt(const unsigned long long* p, unsigned tag, unsigned* err) {
  return __uint_as_float(mg_ldt_u(p, tag, err));
}
// Second half of a batched tagged read: `raw` was loaded from p earlier (several such loads in flight together); only
// a value whose tag has not arrived yet falls back to the bounded wait.
__device__ __forceinline__ unsigned mg_fix_u(const unsigned long long* p, unsigned long long raw, unsigned tag, unsigned* err) {
  if (static_cast<unsigned>(raw >> 32) == tag) return static_cast<unsigned>(raw);
  return mg_wait_tag(p, tag, err);
}
__device__ __forceinline__ float mg_fix(const unsigned long long* p, unsigned long long raw, unsigned tag, unsigned* err) {
  return __uint_as_float(mg_fix_u(p, raw, tag, err));
}
// Batched tagged read of N words: all loads in flight together; while a word is missing, ONE bounded wait on a missing
// word, then the whole batch again. (Fixing the missing words one after the other would cost one L2 round trip per
// word after the data has arrived.) Returns the 32-bit payloads.
template <int N>
__device__ __forceinline__ void mg_read_tagged(const unsigned long long* const (&p)[N], unsigned (&out)[N], unsigned tag, unsigned* err) {
  for (;;) {
    unsigned long long raw[N];
#pragma unroll
    for (int u = 0; u < N; ++u) raw[u] = ld_relaxed_gpu_u64(p[u]);
    const unsigned long long* missing = nullptr;
#pragma unroll
    for (int u = 0; u < N; ++u) {
      out[u] = static_cast<unsigned>(raw[u]);
      if (static_cast<unsigned>(raw[u] >> 32) != tag) missing = p[u];
    }
    if (missing == nullptr) return;
    mg_wait_tag(missing, tag, err);
    if (ld_cg_u(err) != 0u) return;
  }
}

// Shape of a GEMV: 0 = 2 rows x 8 rounds, 1 = 1 x 8, 2 = 2 x 4, 3 = 2 x 2 (rows per warp x 16-byte loads per lane and
// row in flight). Long rows take 8 loads per lane; two rows per warp as soon as a CTA's share of the rows exceeds its
// 16 warps, so that one round of loads covers the share whenever it can.
__device__ __forceinline__ int mg_gemv_shape(int nch, int rows) {
#ifdef MG_ONE_SHAPE
  return 2;
#else
#ifndef MG_R2_WAVES
#define MG_R2_WAVES 1
#endif
  if (nch > 128) return rows > MG_R2_WAVES * static_cast<int>(gridDim.x) * MG_WARPS ? 0 : 1;
  return nch > 64 ? 2 : 3;
#endif
}
__device__ __forceinline__ int mg_gemv_rows_per_warp(int nch, int rows) { return mg_gemv_shape(nch, rows) == 1 ? 1 : 2; }
// Last row of CTA b's contiguous run of a GEMV over `rows` rows (the run may be empty: then the previous run's end).
__device__ __forceinline__ int mg_run_end(int nch, int rows, int b) {
  const int R = mg_gemv_rows_per_warp(nch, rows);
  const unsigned ngroups = static_cast<unsigned>((rows + R - 1) / R);
  const int g1 = static_cast<int>(ngroups * static_cast<unsigned>(b + 1) / gridDim.x);
  return max(0, min(rows, g1 * R) - 1);
}
// Warp 0 polls (bounded) the element at the end of every CTA's run until all carry the tag: the producers' rows are
// then very likely all there, and the batched reads that follow find them at the first attempt. Call with the whole
// CTA; ends with a CTA barrier.
__device__ __forceinline__ void mg_wait_runs_tagged(const unsigned long long* vec, int nch, int rows, unsigned tag, unsigned* err, bool live) {
  if (threadIdx.x < 32 && live) {
    const int nb = static_cast<int>(gridDim.x);
    for (int b0 = 0; b0 < nb; b0 += 128) {
      const unsigned long long* ps[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) ps[u] = vec + mg_run_end(nch, rows, min(b0 + static_cast<int>(threadIdx.x) + 32 * u, nb - 1));
      unsigned bits[4];
      mg_read_tagged<4>(ps, bits, tag, err);
    }
  }
  __syncthreads();
}

// The layer table lives in global memory; its entry for the NEXT layer is copied into shared memory while the current
// layer runs, so that no phase starts with a dependent load of a weight pointer from L2.
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void mg_fetch_layer(IhbMegaLayer* dst, const IhbMegaLayer* src) {
  static_assert(sizeof(IhbMegaLayer) % 16 == 0, "layer entries are copied in 16-byte pieces");
  if (threadIdx.x < sizeof(IhbMegaLayer) / 16)
    cp_async16(reinterpret_cast<char*>(dst) + 16 * threadIdx.x, reinterpret_cast<const char*>(src) + 16 * threadIdx.x);
  asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void mg_fetch_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// End of a phase inside a CTA: shared memory may be reused; the profile gets its stamp.
__device__ __forceinline__ void mg_phase_end(const IhbMegaArgs& a, MgCtx& c, int stamp) {
  mg_fetch_wait();
  __syncthreads();
  mg_stamp(a, stamp);
}

// Stages n values with U per thread and round: f(i, v) fills v[u] for index i + u * MG_THREADS (anything past n is
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
      if (idx < n) mg_stage_put<FP8>(c, idx, v[u], m);
    }
  }
  mg_stage_finish<FP8>(c, n, m);
}

// resid (+= scale * the all-reduce round pushed last) -> RMSNorm(gamma) -> xf (fp32) and the staged GEMV input: one
// pass that adds the slots and collects both reductions (sum of squares; maximum for the fp16 pre-scale) with one
// pair of CTA barriers, one pass that writes the normed vector. ONE thread first polls the slot of the last row
// (written in a rank's last GEMV wave) while the others sleep at a barrier: 75 000 threads polling L2 would slow the
// CTAs that are still streaming weights. Then every thread reads its slots (two groups of four in flight) and spins
// only on those that are not complete yet.
template <bool FP8>
__device__ __noinline__ float mg_residual_norm_fn(const IhbMegaArgs* ap, unsigned epoch, unsigned ar_n, int add_slots,
                                                 const float* gamma, float scale, int stamp, int push_nch) {
  const IhbMegaArgs& a = *ap;
  MgCtx c;
  mg_ctx_pointers<FP8>(a, c);
  c.epoch = epoch;
  c.ar_n = ar_n;
  constexpr int NIT = 2;                       // float4 groups per thread and round
  const int H = a.H, tid = threadIdx.x;
  float ss = 0.f, mx = 0.f;
  const unsigned long long* base = nullptr;
  const unsigned n = c.ar_n;
  bool ok = c.flags[0] == 0;
  if (add_slots && a.delay_ns > 0 && static_cast<int>(blockIdx.x) == a.delay_cta) {
    // test aid: this CTA lags (bounded) before it reads the round; everything else has to cope
    const unsigned long long t0 = globaltimer_ns();
    const unsigned long long lim = static_cast<unsigned long long>(min(a.delay_ns, 1000000));
    while (globaltimer_ns() - t0 < lim) { }
  }
  if (add_slots) {
    // c.epoch - 1: the round that ended with the last push
    base = reinterpret_cast<const unsigned long long*>(a.comm.slots_local) + static_cast<size_t>((c.epoch - 1u) & (MG_NPAR - 1)) * H;
    if (tid < 32 && ok) {
      // sentinels: the slot of the last row of every CTA's run of the H-row GEMV that pushed this round (push_nch
      // tells its shape); complete there means complete nearly everywhere
      const int nb = static_cast<int>(gridDim.x);
      const unsigned long long* ps[8];                       // up to 256 CTAs
#pragma unroll
      for (int u = 0; u < 8; ++u) ps[u] = base + mg_run_end(push_nch, H, min(tid + 32 * u, nb - 1));
      const unsigned long long t0 = globaltimer_ns();
      unsigned spins = 0;
      for (;;) {
        unsigned long long w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) w[u] = (32 * u < nb) ? ld_relaxed_sys_u64(ps[u]) : 0ull;
        bool all = true;
#pragma unroll
        for (int u = 0; u < 8; ++u) all = all && (32 * u >= nb || static_cast<unsigned>(w[u] >> 56) == n);
        if (__all_sync(0xffffffffu, all)) break;
        if ((++spins & 63u) == 0u) {
          bool stop = ld_cg_u(a.err) != 0u;
          if (!stop && globaltimer_ns() - t0 > IHB_PEER_WAIT_NS) { set_error(a.err, ERR_PEER_BARRIER_TIMEOUT); stop = true; }
          if (__any_sync(0xffffffffu, stop)) break;
        }
      }
    }
    __syncthreads();
  }
  for (int i0 = 0; i0 < H; i0 += NIT * MG_THREADS * 4) {
    float4 v[NIT];
    if (add_slots) {
      ulonglong2 p[NIT][2];
      for (;;) {
        const unsigned long long* missing = nullptr;
#pragma unroll
        for (int it = 0; it < NIT; ++it) {
          const int i = i0 + (tid + it * MG_THREADS) * 4;
          if (i < H) { p[it][0] = ld_relaxed_sys_v2_u64(base + i); p[it][1] = ld_relaxed_sys_v2_u64(base + i + 2); }
        }
#pragma unroll
        for (int it = 0; it < NIT; ++it) {
          const int i = i0 + (tid + it * MG_THREADS) * 4;
          if (i < H && !mg_counted(p[it], n)) missing = base + i;
        }
        if (missing == nullptr || !ok) break;
        ok = mg_wait_counted(missing, n, a.err);
      }
#pragma unroll
      for (int it = 0; it < NIT; ++it) {
        const int i = i0 + (tid + it * MG_THREADS) * 4;
        if (i < H) {
          const float4 r = *reinterpret_cast<const float4*>(c.resid + i);
          v[it] = make_float4(fmaf(mg_decode(p[it][0].x, n), scale, r.x), fmaf(mg_decode(p[it][0].y, n), scale, r.y),
                              fmaf(mg_decode(p[it][1].x, n), scale, r.z), fmaf(mg_decode(p[it][1].y, n), scale, r.w));
          *reinterpret_cast<float4*>(c.resid + i) = v[it];
        }
      }
    } else {
#pragma unroll
      for (int it = 0; it < NIT; ++it) {
        const int i = i0 + (tid + it * MG_THREADS) * 4;
        if (i < H) v[it] = *reinterpret_cast<const float4*>(c.resid + i);
      }
    }
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int i = i0 + (tid + it * MG_THREADS) * 4;
      if (i < H) {
        const float4 g = *reinterpret_cast<const float4*>(gamma + i);
        ss += v[it].x * v[it].x + v[it].y * v[it].y + v[it].z * v[it].z + v[it].w * v[it].w;
        mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v[it].x * g.x), fabsf(v[it].y * g.y))), fmaxf(fabsf(v[it].z * g.z), fabsf(v[it].w * g.w)));
      }
    }
  }
  const float2 tot = block_sum_max(ss, mx, c.red);
  if (add_slots) mg_stamp(a, stamp);
  const float rinv = rsqrtf(tot.x / static_cast<float>(H) + a.eps);
  float ps = 1.f;
  c.unscale = 1.f;
  if (FP8 && tot.y * rinv > 8.f) {
    const int e = static_cast<int>(ceilf(log2f(tot.y * rinv * 0.125f)));
    ps = exp2f(static_cast<float>(-e));
    c.unscale = exp2f(static_cast<float>(e));
  }
  // every thread reads back the elements it wrote itself
  for (int i = tid * 4; i < H; i += MG_THREADS * 4) {
    const float4 r = *reinterpret_cast<const float4*>(c.resid + i);
    const float4 g = *reinterpret_cast<const float4*>(gamma + i);
    const float4 x = make_float4(r.x * g.x * rinv, r.y * g.y * rinv, r.z * g.z * rinv, r.w * g.w * rinv);
    *reinterpret_cast<float4*>(c.xf + i) = x;
    if (FP8) {
      *reinterpret_cast<__half2*>(c.xh + i) = __floats2half2_rn(x.x * ps, x.y * ps);
      *reinterpret_cast<__half2*>(c.xh + i + 2) = __floats2half2_rn(x.z * ps, x.w * ps);
    } else {
      *reinterpret_cast<float4*>(c.xv + i) = x;
    }
  }
  __syncthreads();
  return c.unscale;
}
template <bool FP8>
__device__ __forceinline__ void mg_residual_norm(const IhbMegaArgs& a, MgCtx& c, bool add_slots, const float* gamma,
                                                 float scale, int stamp, int push_nch) {
  c.unscale = mg_residual_norm_fn<FP8>(&a, c.epoch, c.ar_n, add_slots ? 1 : 0, gamma, scale, stamp, push_nch);
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
// Row groups are dealt to the CTAs in equal contiguous runs (every CTA streams one contiguous piece of the matrix
// and, with at least as many groups as CTAs, every CTA produces rows); the warps of a CTA interleave inside the run.
enum { MG_PLAIN = 0, MG_EXPERT = 1, MG_DOWN = 2 };
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

// Returns the packed running maximum of this warp's rows (ARGMAX sink; valid in lane 0).
template <bool FP8, int R, int U>
__device__ __forceinline__ unsigned long long mg_gemv(const IhbMegaArgs& a, const MgPlan& plan, const MgSink& sink,
                                                      const __half* xh, const float* xv, float unscale_in,
                                                      const int* flags) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long best = 0ull;
  const int n = plan.rows, nch = plan.nch, kbs = plan.kbs;
  const int ngroups = (n + R - 1) / R;
  // ngroups * gridDim < 2^31 (rows < 2^22, at most a few hundred CTAs)
  const int g0 = static_cast<int>(static_cast<unsigned>(ngroups) * blockIdx.x / gridDim.x);
  const int g1 = static_cast<int>(static_cast<unsigned>(ngroups) * (blockIdx.x + 1u) / gridDim.x);
  const float unscale = FP8 ? unscale_in : 1.f;
  const bool down = plan.kind == MG_DOWN;
  for (int g = g0 + warp; g < g1; g += MG_WARPS) {
    const int i0 = g * R;
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
    // lane j keeps row j's sum: the sink code exists once and the R results leave together
    float v = 0.f;
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const float t = warp_sum(acc[j]);
      if (lane == j) v = t;
    }
    v *= unscale;
    const int i = i0 + lane;
    if (lane < R && i < n) {
      if (sink.kind == MG_STORE) {
        st_relaxed_gpu_u64(reinterpret_cast<unsigned long long*>(sink.out) + i,
                           mg_pack(v, static_cast<unsigned>(*reinterpret_cast<const volatile int*>(flags + 3))));
      } else if (sink.kind == MG_PUSH) {
        mg_push(a, sink.off + i, v);
      } else {
        const unsigned long long pk = pack_max(v, static_cast<unsigned>(i));
        best = pk > best ? pk : best;
        if (sink.out != nullptr) sink.out[i] = v;
      }
    }
  }
  if (sink.kind == MG_ARGMAX) {
#pragma unroll
    for (int o = 1; o < R; o <<= 1) {
      const unsigned long long q = __shfl_xor_sync(0xffffffffu, best, o);
      best = q > best ? q : best;
    }
  }
  return best;
}

// The GEMV whose plan and sink thread 0 put into shared memory before the last CTA barrier. Picks the (rows, rounds)
// shape by the number of chunk rounds a row needs and by how many rows a warp gets. Compiled once, out of line.
template <bool FP8>
__device__ __noinline__ unsigned long long mg_gemv_run(const IhbMegaArgs* ap, float unscale) {
  const IhbMegaArgs& a = *ap;
  MgCtx c;
  mg_ctx_pointers<FP8>(a, c);
  MgPlan plan = mg_shm().plan;
  const MgSink sink = mg_shm().sink;
  // the two shared-memory operands of a plan are always these
  plan.sel_e = c.sel_e;
  plan.tab = reinterpret_cast<const uint2*>(c.attn);
  const __half* xh = c.xh;
  const float* xv = c.xv;
  const int* flags = c.flags;
#ifdef MG_ONE_SHAPE
  return mg_gemv<FP8, 2, 4>(a, plan, sink, xh, xv, unscale, flags);
#else
  switch (mg_gemv_shape(plan.nch, plan.rows)) {
    case 0: return mg_gemv<FP8, 2, 8>(a, plan, sink, xh, xv, unscale, flags);
    case 1: return mg_gemv<FP8, 1, 8>(a, plan, sink, xh, xv, unscale, flags);
    case 2: return mg_gemv<FP8, 2, 4>(a, plan, sink, xh, xv, unscale, flags);
    default: return mg_gemv<FP8, 2, 2>(a, plan, sink, xh, xv, unscale, flags);
  }
#endif
}
// Publishes the arguments of the next GEMV; a CTA barrier must follow before mg_gemv_run.
__device__ __forceinline__ void mg_gemv_args(const MgPlan& pl, int sink_kind, float* out, size_t off) {
  if (threadIdx.x == 0) {
    MgShm& sh = mg_shm();
    sh.plan = pl;
    sh.sink.kind = sink_kind; sh.sink.out = out; sh.sink.off = off;
  }
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

#include "mega_attn.inc"
#include "mega_phases.inc"

}  // namespace ihb

#include "mega_host.inc"
