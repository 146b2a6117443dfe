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

constexpr int MG_THREADS = 256;
constexpr int MG_WARPS = 8;
constexpr int MG_HD = 128;
constexpr int MG_GQ = 8;                 // query heads per attention work item
constexpr int MG_REC = MG_HD + 2;        // attention partial record: acc[128], m, l

struct MgAttnSmem {
  float q[MG_GQ][MG_HD];
  float p[MG_WARPS][MG_GQ][32];
  float m[MG_WARPS][MG_GQ], l[MG_WARPS][MG_GQ];
  float acc[MG_WARPS][MG_GQ][MG_HD];
  __nv_bfloat16 knew[MG_HD], vnew[MG_HD];
};

struct MgCtx {
  // barrier state: the counters are meaningful in thread 0; epoch (cross-GPU rounds so far) in every thread
  unsigned base, rel_base, n_bar, n_rel, epoch;
  // shared memory carve-up
  float* resid;          // [H]
  float* xf;             // fp32 activation vector (router input; every GEMV input for bf16 weights)
  __half* xh;            // fp16 pre-scaled activation vector (fp8 weights)
  float* red;            // [32] block reductions
  int* sel_e;            // [top_k]
  float* sel_w;          // [top_k]
  int* flags;            // [0] dead, [1] last-arriver flag of the attention merge
  MgAttnSmem* attn;
  uint8_t* ring;         // [warps][MG_STAGES][4 KB] weight stream
  float unscale;         // undoes the power-of-two pre-scale of xh
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

// Grid-wide barrier: one fire-and-forget release-add per CTA, then a spin on the same counter. cross = true:
// CTA 0, once every CTA of this GPU has arrived (all partials pushed), also runs the cross-GPU arrive/wait and
// then opens a second counter on which the other CTAs wait.
__device__ __forceinline__ void mg_barrier(const IhbMegaArgs& a, MgCtx& c, bool cross) {
  __syncthreads();
  if (threadIdx.x == 0 && c.flags[0] == 0) {
    c.n_bar++;
    const unsigned target = c.base + c.n_bar * gridDim.x;
    bool ok = true;
    if (cross && a.comm.nranks > 1) {
      __threadfence_system();
      red_release_gpu_add_u32(a.bar + 0, 1u);
      c.n_rel++;
      if (blockIdx.x == 0) {
        ok = mg_wait(a.bar + 0, target, a.err);
        ok = ok && peer_barrier(a.comm, (c.epoch + 1u) * static_cast<unsigned>(a.comm.nranks), a.err);
        red_release_gpu_add_u32(a.bar + 1, 1u);
      } else {
        ok = mg_wait(a.bar + 1, c.rel_base + c.n_rel, a.err);
      }
    } else {
      red_release_gpu_add_u32(a.bar + 0, 1u);
      ok = mg_wait(a.bar + 0, target, a.err);
    }
    if (!ok) c.flags[0] = 1;
    if (a.prof != nullptr && blockIdx.x == 0) a.prof[c.n_bar] = globaltimer_ns();
  }
  if (cross) c.epoch++;          // every thread keeps the count of cross-GPU rounds (it selects the slot parity)
  __syncthreads();
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

// xf[0..n) (fp32, shared) -> xh (fp16, shared) scaled by a power of two so that max|x| <= 8 (bounds the fp16
// accumulation chains of dot16_e4m3); c.unscale undoes it.
__device__ __forceinline__ void mg_stage_half(MgCtx& c, const float* src, int n) {
  float m = 0.f;
  for (int i = threadIdx.x; i < n; i += MG_THREADS) m = fmaxf(m, fabsf(src[i]));
  m = block_max(m, c.red);
  int e = 0;
  if (m > 8.f) e = static_cast<int>(ceilf(log2f(m * 0.125f)));
  const float s = exp2f(static_cast<float>(-e));
  c.unscale = exp2f(static_cast<float>(e));
  for (int i = threadIdx.x; i < n; i += MG_THREADS) c.xh[i] = __float2half_rn(src[i] * s);
  __syncthreads();
}

// n values produced by f(i) (one global read each) -> xh: stored as fp16 at once, the maximum is found on the way and
// the vector is re-scaled in shared memory only when it exceeds 8 (a power-of-two factor: no second rounding).
template <typename F>
__device__ __forceinline__ void mg_stage_half_from(MgCtx& c, int n, F f) {
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
    const __half s = __float2half_rn(exp2f(static_cast<float>(-e)));
    c.unscale = exp2f(static_cast<float>(e));
    for (int i = threadIdx.x; i < n; i += MG_THREADS) c.xh[i] = __hmul(c.xh[i], s);
  }
  __syncthreads();
}

// resid (+= the all-reduce slots of `parity`, in rank order) -> RMSNorm(gamma) -> xf (fp32) [+ xh].
__device__ __forceinline__ void mg_residual_norm(const IhbMegaArgs& a, MgCtx& c, bool add_slots, int parity,
                                                 const float* gamma, bool want_half) {
  const int H = a.H;
  const int nr = a.comm.nranks;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < H; i += MG_THREADS * 4) {
    float4 v = *reinterpret_cast<float4*>(c.resid + i);
    if (add_slots) {
      const float* sl = a.comm.slots_local + static_cast<size_t>(parity) * nr * H + i;
      for (int r = 0; r < nr; ++r) {
        const float4 p = ld_cg_f4(reinterpret_cast<const float4*>(sl + static_cast<size_t>(r) * H));
        v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
      }
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
  if (want_half) mg_stage_half(c, c.xf, H);
}

// ---- streaming GEMV building block --------------------------------------------------------------------------------------------
// Every warp owns a private ring of MG_STAGES x 4 KB in shared memory that its lanes fill with 16-byte asynchronous
// copies (cp.async: the bytes in flight live in shared memory, not in registers - up to 128 KB per SM, enough to
// cover HBM latency at full bandwidth; bulk TMA copies of this size are bound by their issue rate instead). Work is dealt in groups of R consecutive output rows; a group is streamed as P contiguous pieces of
// at most 4 KB (R whole short rows, or one slice of a long row, or - for the down projection - R rows of one
// routed expert). Chunk = 16 bytes of weights = EPC activation elements (16 for e4m3, 8 for bf16).
constexpr int MG_STAGES = 3;
constexpr int MG_STAGE_BYTES = 4096;

struct Piece {
  const uint8_t* src;    // first byte (16-byte aligned)
  unsigned bytes;        // nr * seg
  int seg;               // bytes of one row inside the piece
  int nr;                // rows in the piece (<= R)
  int xchunk0;           // first activation chunk this piece multiplies
  int kc0;               // chunk offset inside the (expert's) row, for the block-scale column
  const float* srow;     // scale row of the piece's rows (all R rows share a row block)
  int out0;              // output index of row 0
};

struct PlainPlan {
  const uint8_t* W; const float* sc; int rows, rowbytes, rb, kbs, nkb, R, P, seg;
  __device__ __forceinline__ Piece piece(int g, int p) const {
    Piece pc;
    const int r0 = g * R;
    pc.nr = min(R, rows - r0);
    pc.seg = seg;
    pc.src = W + static_cast<size_t>(r0) * rowbytes + static_cast<size_t>(p) * seg;
    pc.bytes = static_cast<unsigned>(pc.nr) * seg;
    pc.xchunk0 = pc.kc0 = (p * seg) >> 4;
    pc.srow = sc + static_cast<size_t>(r0 / rb) * nkb;
    pc.out0 = r0;
    return pc;
  }
};
// gate / up: virtual row v = slot * rpe + jj (rpe = 2 I rows per expert)
struct ExpertPlan {
  const uint8_t* W; const float* sc; int rowbytes, rb, kbs, nkb, R, P, seg, rpe, nrb; const int* sel_e;
  __device__ __forceinline__ Piece piece(int g, int p) const {
    Piece pc;
    const int v0 = g * R;
    const int slot = v0 / rpe, jj0 = v0 - slot * rpe;
    const size_t e = static_cast<size_t>(sel_e[slot]);
    pc.nr = R;
    pc.seg = seg;
    pc.src = W + (e * rpe + jj0) * rowbytes + static_cast<size_t>(p) * seg;
    pc.bytes = static_cast<unsigned>(R) * seg;
    pc.xchunk0 = pc.kc0 = (p * seg) >> 4;
    pc.srow = sc + (e * nrb + jj0 / rb) * nkb;
    pc.out0 = v0;
    return pc;
  }
};
// down: group = R consecutive output rows, piece p = routing slot p (R rows of that expert, contiguous)
struct DownPlan {
  const uint8_t* W; const float* sc; int rowbytes, rb, kbs, nkb, R, nch1, H, nrb; const int* sel_e;
  __device__ __forceinline__ Piece piece(int g, int p) const {
    Piece pc;
    const int r0 = g * R;
    const size_t e = static_cast<size_t>(sel_e[p]);
    pc.nr = min(R, H - r0);
    pc.seg = rowbytes;
    pc.src = W + (e * H + r0) * rowbytes;
    pc.bytes = static_cast<unsigned>(pc.nr) * rowbytes;
    pc.xchunk0 = p * nch1;
    pc.kc0 = 0;
    pc.srow = sc + (e * nrb + r0 / rb) * nkb;
    pc.out0 = r0;
    return pc;
  }
};

template <bool FP8>
__device__ __forceinline__ float mg_chunk_dot(uint4 w, const MgCtx& c, int cch) {
  if (FP8) {
    const uint4* x = reinterpret_cast<const uint4*>(c.xh + 16 * cch);
    return dot16_e4m3(w, x[0], x[1]);
  } else {
    const float4* x = reinterpret_cast<const float4*>(c.xf + 8 * cch);
    return dot8_bf16(w, x[0], x[1]);
  }
}

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// sink(output index, value) is called by one lane per finished row.
template <bool FP8, int R, typename Plan, typename Sink>
__device__ __forceinline__ void mg_stream(const IhbMegaArgs& a, MgCtx& c, const Plan& plan, int ngroups, int P, int kbs,
                                          Sink sink) {
  if (c.flags[0] != 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gw = warp * gridDim.x + blockIdx.x;      // consecutive groups go to different SMs
  const int W = gridDim.x * MG_WARPS;
  const int mine = ngroups > gw ? (ngroups - gw + W - 1) / W : 0;
  const int total = mine * P;
  uint8_t* ring = c.ring + warp * (MG_STAGES * MG_STAGE_BYTES);
  // every lane copies its 16-byte chunks of the piece (asynchronous, no registers held); one commit group per piece,
  // committed even when empty so that "at most MG_STAGES - 1 groups pending" always means "piece t has landed"
  auto issue = [&](int t) {
    if (t < total) {
      const Piece pc = plan.piece(gw + (t / P) * W, t % P);
      uint8_t* dst = ring + (t % MG_STAGES) * MG_STAGE_BYTES;
      const int nch = static_cast<int>(pc.bytes >> 4);
#pragma unroll 4
      for (int cc = lane; cc < nch; cc += 32) cp_async16(dst + 16 * cc, pc.src + 16 * cc);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int t = 0; t < MG_STAGES - 1; ++t) issue(t);
  float acc[R];
  for (int t = 0; t < total; ++t) {
    issue(t + MG_STAGES - 1);                      // its stage was consumed in iteration t - 1
    const int p = t % P;
    const Piece pc = plan.piece(gw + (t / P) * W, p);
    if (p == 0) {
#pragma unroll
      for (int j = 0; j < R; ++j) acc[j] = 0.f;
    }
    cp_async_wait<MG_STAGES - 1>();
    __syncwarp();                                  // the other lanes' chunks of piece t are visible too
    const uint8_t* sm = ring + (t % MG_STAGES) * MG_STAGE_BYTES;
    const int segch = pc.seg >> 4;
#pragma unroll
    for (int j = 0; j < R; ++j) {
      if (j < pc.nr) {
        const uint8_t* row = sm + j * pc.seg;
#pragma unroll 4
        for (int cc = lane; cc < segch; cc += 32) {
          const uint4 w = *reinterpret_cast<const uint4*>(row + 16 * cc);
          const float s = FP8 ? __ldg(pc.srow + ((pc.kc0 + cc) >> kbs)) : 1.f;
          acc[j] = fmaf(s, mg_chunk_dot<FP8>(w, c, pc.xchunk0 + cc), acc[j]);
        }
      }
    }
    __syncwarp();                                  // all lanes are done with this stage before it is refilled
    if (p == P - 1) {
#pragma unroll
      for (int j = 0; j < R; ++j) {
        const float v = warp_sum(acc[j]) * (FP8 ? c.unscale : 1.f);
        if (lane == (j & 31) && j < pc.nr) sink(pc.out0 + j, v);
      }
    }
  }
  cp_async_wait<0>();
}

template <bool FP8, typename Plan, typename Sink>
__device__ __forceinline__ void mg_stream_auto(const IhbMegaArgs& a, MgCtx& c, const Plan& plan, int R, int ngroups, int P,
                                               int kbs, Sink sink) {
  if (R == 1) mg_stream<FP8, 1>(a, c, plan, ngroups, P, kbs, sink);
  else if (R == 2) mg_stream<FP8, 2>(a, c, plan, ngroups, P, kbs, sink);
  else if (R == 4) mg_stream<FP8, 4>(a, c, plan, ngroups, P, kbs, sink);
  else mg_stream<FP8, 16>(a, c, plan, ngroups, P, kbs, sink);
}

// Rows per group for rows of `rowbytes` bytes: as many whole rows as fit a 4 KB stage (1, 2, 4 or 16), but no more
// than keeps every warp of the grid busy (short serial chains matter more than long copies when a matrix is small),
// and never straddling a scale row block (`rb`) or `align` rows.
__device__ __forceinline__ int mg_rows_per_group(int rowbytes, int rb, int align, int rows) {
  int R = 1;
  const int fit = MG_STAGE_BYTES / rowbytes;
  const int W = gridDim.x * MG_WARPS;
  if (fit >= 16) R = 16; else if (fit >= 4) R = 4; else if (fit >= 2) R = 2;
  while (R > 1 && ((rb % R) != 0 || (align % R) != 0 || rows / R < W)) R = (R == 16) ? 4 : R / 2;
  return R;
}

__device__ __forceinline__ PlainPlan plain_plan(const IhbMat& m, bool fp8) {
  PlainPlan pl;
  pl.W = m.W; pl.sc = m.wscale; pl.rows = m.rows; pl.rowbytes = fp8 ? m.K : 2 * m.K;
  pl.rb = m.rb > 0 ? m.rb : (1 << 30); pl.kbs = m.kb_shift; pl.nkb = m.nkb;
  if (pl.rowbytes > MG_STAGE_BYTES) {
    pl.R = 1; pl.seg = MG_STAGE_BYTES; pl.P = pl.rowbytes / MG_STAGE_BYTES;     // rows are multiples of 4 KB (checked on the host)
  } else {
    pl.R = mg_rows_per_group(pl.rowbytes, pl.rb == (1 << 30) ? 16 : pl.rb, 16, pl.rows); pl.seg = pl.rowbytes; pl.P = 1;
  }
  return pl;
}

#include "mega_phases.inc"

}  // namespace ihb

#include "mega_host.inc"
