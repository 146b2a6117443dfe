// Stand-alone fused all-reduce (+ residual + RMSNorm) over symmetric memory, for hidden-state tensors [T, H] from
// 8 KB (one token) to tens of MB (prefill chunks), and for the collective sweep.
//
//   one-shot  every rank pushes its whole input into slot `rank` of every GPU (multimem.st through NVSwitch, or one
//             store per peer), one cross-GPU arrive/wait, every rank adds the slots in rank order (bitwise identical
//             results on all ranks) and applies residual + RMSNorm itself. Latency-optimal for small messages: the
//             data crosses NVLink once and there is a single barrier.
//   two-shot  rows are dealt to ranks; the owner of a row reduces it - multimem.ld_reduce lets the switch add the
//             row of all GPUs in flight (NVLS), else peer loads added in rank order - adds the residual, normalises,
//             and broadcasts the finished row (multimem.st or peer stores). Bandwidth-optimal for large messages:
//             each GPU moves 2 (n - 1) / n of the data instead of n - 1 times.
// Both run as ONE kernel launch with bounded waits. The reference keeps the reduction and the norm in separate
// kernels (kernels/nvls_engine.cuh:160-200 then tp8_residual_rmsnorm_quant, kernels/decode_step_tp8.cu:693-718) and
// has a one-shot P2P variant without norm (kernels/oneshot_allreduce.cu:123-196).
#include "common.cuh"
#include "tails.cuh"

namespace ihb {

struct ArArgs {
  IhbComm comm;          // slots region: one-shot [2][nranks][T * H]; two-shot: IN [T * H] then OUT [T * H] (fp32)
  const float* x;        // [T, H] this rank's partial (fp32)
  const float* resid;    // optional [T, H]
  const float* gamma;    // optional [H]: RMSNorm weight (NULL: plain all-reduce)
  float* out;            // [T, H] reduced (+ residual) rows
  float* out_norm;       // optional [T, H]
  void* out_norm_bf16;   // optional [T, H] bf16: the normed rows rounded for a tensor-core GEMM that follows
  float eps;
  int T, H;
  unsigned* counter;     // grid arrival counter (zero before the first launch)
  unsigned* err;
};

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All CTAs of this GPU arrive, CTA 0 runs the cross-GPU round, everyone leaves. `round` counts rounds within the launch.
__device__ __forceinline__ bool ar_grid_peer_barrier(const ArArgs& a, unsigned epoch, unsigned round) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    bool ok = true;
    const unsigned base = ld_cg_u(a.counter + 2);
    __threadfence_system();
    atomicAdd(a.counter + 0, 1u);
    const unsigned t0 = base + (round + 1u) * gridDim.x;
    if (blockIdx.x == 0) {
      const unsigned long long st = globaltimer_ns();
      while (static_cast<int>(ld_acquire_gpu(a.counter + 0) - t0) < 0)
        if (globaltimer_ns() - st > IHB_LOCAL_WAIT_NS) { set_error(a.err, ERR_GRID_COUNTER_TIMEOUT); ok = false; break; }
      if (ok && a.comm.nranks > 1) ok = peer_barrier(a.comm, (epoch + 1u) * static_cast<unsigned>(a.comm.nranks), a.err);
      __threadfence();
      atomicAdd(a.counter + 1, 1u);
    }
    const unsigned rbase = ld_cg_u(a.counter + 3);
    const unsigned long long st = globaltimer_ns();
    while (static_cast<int>(ld_acquire_gpu(a.counter + 1) - (rbase + round + 1u)) < 0)
      if (globaltimer_ns() - st > IHB_LOCAL_WAIT_NS + IHB_PEER_WAIT_NS) { set_error(a.err, ERR_GRID_COUNTER_TIMEOUT); ok = false; break; }
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  return s_ok != 0;
}

// residual + RMSNorm of one row held as float4s strided over the CTA
template <int NTHR>
__device__ __forceinline__ void ar_finish_row(const ArArgs& a, int t, float4* v, int nv, float* red) {
  const int H = a.H;
  float ss = 0.f;
  for (int j = 0; j < nv; ++j) {
    const int i = (threadIdx.x + NTHR * j) * 4;
    if (i < H) {
      if (a.resid != nullptr) {
        const float4 r = *reinterpret_cast<const float4*>(a.resid + static_cast<size_t>(t) * H + i);
        v[j].x += r.x; v[j].y += r.y; v[j].z += r.z; v[j].w += r.w;
      }
      ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
    }
  }
  if (a.gamma == nullptr) return;
  ss = warp_sum(ss);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < NTHR / 32; ++w) tot += red[w];
  const float rinv = rsqrtf(tot / static_cast<float>(H) + a.eps);
  for (int j = 0; j < nv; ++j) {
    const int i = (threadIdx.x + NTHR * j) * 4;
    if (i < H && (a.out_norm != nullptr || a.out_norm_bf16 != nullptr)) {
      const float4 g = *reinterpret_cast<const float4*>(a.gamma + i);
      const float4 y = make_float4(v[j].x * rinv * g.x, v[j].y * rinv * g.y, v[j].z * rinv * g.z, v[j].w * rinv * g.w);
      if (a.out_norm != nullptr) *reinterpret_cast<float4*>(a.out_norm + static_cast<size_t>(t) * H + i) = y;
      if (a.out_norm_bf16 != nullptr) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.out_norm_bf16) + static_cast<size_t>(t) * H + i) =
            make_uint2(*reinterpret_cast<const unsigned*>(&lo), *reinterpret_cast<const unsigned*>(&hi));
      }
    }
  }
}

constexpr int AR_THREADS = 256;
constexpr int AR_MAXV = 8;            // H <= 8192

__global__ void __launch_bounds__(AR_THREADS) ar_oneshot_kernel(const ArArgs a) {
  __shared__ float red[AR_THREADS / 32];
  const IhbComm& cm = a.comm;
  const unsigned epoch = *cm.epoch;
  const int parity = epoch & 1u;
  const size_t n = static_cast<size_t>(a.T) * a.H;
  // push this rank's rows into slot `rank` everywhere
  const size_t slot0 = (static_cast<size_t>(parity) * cm.nranks + cm.rank) * n;
  for (size_t i = (static_cast<size_t>(blockIdx.x) * AR_THREADS + threadIdx.x) * 4; i < n;
       i += static_cast<size_t>(gridDim.x) * AR_THREADS * 4) {
    const float4 v = *reinterpret_cast<const float4*>(a.x + i);
    if (cm.nranks == 1) {
      *reinterpret_cast<float4*>(cm.slots_local + slot0 + i) = v;
    } else if (cm.slots_mc != nullptr) {
      multimem_st_f4(cm.slots_mc + slot0 + i, v);
    } else {
      for (int p = 0; p < cm.nranks; ++p) {
        float* d = cm.slots_peer[p] + slot0 + i;
        asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(d), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
      }
    }
  }
  const bool ok = ar_grid_peer_barrier(a, epoch, 0);
  if (ok) {
    const float* slots = cm.slots_local + static_cast<size_t>(parity) * cm.nranks * n;
    for (int t = blockIdx.x; t < a.T; t += gridDim.x) {
      float4 v[AR_MAXV];
      for (int j = 0; j < AR_MAXV; ++j) {
        const int i = (threadIdx.x + AR_THREADS * j) * 4;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < a.H)
          for (int r = 0; r < cm.nranks; ++r) {
            const float4 p = ld_cg_f4(reinterpret_cast<const float4*>(slots + static_cast<size_t>(r) * n + static_cast<size_t>(t) * a.H + i));
            v[j].x += p.x; v[j].y += p.y; v[j].z += p.z; v[j].w += p.w;
          }
      }
      ar_finish_row<AR_THREADS>(a, t, v, AR_MAXV, red);
      for (int j = 0; j < AR_MAXV; ++j) {
        const int i = (threadIdx.x + AR_THREADS * j) * 4;
        if (i < a.H) *reinterpret_cast<float4*>(a.out + static_cast<size_t>(t) * a.H + i) = v[j];
      }
    }
  }
  // bookkeeping for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned done = atomicAdd(a.counter + 4, 1u);
    if (done == gridDim.x - 1) {
      a.counter[4] = 0u;
      a.counter[2] += gridDim.x;
      a.counter[3] += 1u;
      *cm.epoch = epoch + 1u;
      __threadfence();
    }
  }
}

// two-shot: IN = slots[0 .. n), OUT = slots[n .. 2 n) of every GPU's symmetric buffer
__global__ void __launch_bounds__(AR_THREADS) ar_twoshot_kernel(const ArArgs a) {
  __shared__ float red[AR_THREADS / 32];
  const IhbComm& cm = a.comm;
  const unsigned epoch = *cm.epoch;
  const size_t n = static_cast<size_t>(a.T) * a.H;
  for (size_t i = (static_cast<size_t>(blockIdx.x) * AR_THREADS + threadIdx.x) * 4; i < n;
       i += static_cast<size_t>(gridDim.x) * AR_THREADS * 4)
    *reinterpret_cast<float4*>(cm.slots_local + i) = *reinterpret_cast<const float4*>(a.x + i);
  bool ok = ar_grid_peer_barrier(a, epoch, 0);                 // every rank's input is in place
  if (ok) {
    // rows owned by this rank, dealt over its CTAs
    for (int t = cm.rank + cm.nranks * blockIdx.x; t < a.T; t += cm.nranks * gridDim.x) {
      float4 v[AR_MAXV];
      for (int j = 0; j < AR_MAXV; ++j) {
        const int i = (threadIdx.x + AR_THREADS * j) * 4;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < a.H) {
          const size_t off = static_cast<size_t>(t) * a.H + i;
          if (cm.nranks == 1) {
            v[j] = *reinterpret_cast<const float4*>(cm.slots_local + off);
          } else if (cm.slots_mc != nullptr) {
            v[j] = multimem_ld_reduce_f4(cm.slots_mc + off);     // the switch adds the row of all GPUs
          } else {
            for (int r = 0; r < cm.nranks; ++r) {
              const float4 p = ld_cg_f4(reinterpret_cast<const float4*>(cm.slots_peer[r] + off));
              v[j].x += p.x; v[j].y += p.y; v[j].z += p.z; v[j].w += p.w;
            }
          }
        }
      }
      // the residual is replicated, so the owner finishes the row (residual + norm) before broadcasting it
      ar_finish_row<AR_THREADS>(a, t, v, AR_MAXV, red);
      for (int j = 0; j < AR_MAXV; ++j) {
        const int i = (threadIdx.x + AR_THREADS * j) * 4;
        if (i < a.H) {
          const size_t off = n + static_cast<size_t>(t) * a.H + i;
          if (cm.nranks == 1) {
            *reinterpret_cast<float4*>(cm.slots_local + off) = v[j];
          } else if (cm.slots_mc != nullptr) {
            multimem_st_f4(cm.slots_mc + off, v[j]);
          } else {
            for (int p = 0; p < cm.nranks; ++p) {
              float* d = cm.slots_peer[p] + off;
              asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(d), "f"(v[j].x), "f"(v[j].y), "f"(v[j].z), "f"(v[j].w) : "memory");
            }
          }
        }
      }
    }
  }
  ok = ar_grid_peer_barrier(a, epoch + 1u, 1) && ok;           // every row has been broadcast
  if (ok) {
    const float* src = cm.slots_local + n;
    for (int t = blockIdx.x; t < a.T; t += gridDim.x) {
      float4 v[AR_MAXV];
      for (int j = 0; j < AR_MAXV; ++j) {
        const int i = (threadIdx.x + AR_THREADS * j) * 4;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < a.H) v[j] = ld_cg_f4(reinterpret_cast<const float4*>(src + static_cast<size_t>(t) * a.H + i));
      }
      for (int j = 0; j < AR_MAXV; ++j) {
        const int i = (threadIdx.x + AR_THREADS * j) * 4;
        if (i < a.H) *reinterpret_cast<float4*>(a.out + static_cast<size_t>(t) * a.H + i) = v[j];
      }
      // the owner normalised its rows; the others repeat the (cheap, local) norm on the broadcast sums
      if (a.gamma != nullptr && (a.out_norm != nullptr || a.out_norm_bf16 != nullptr) && (t % cm.nranks) != cm.rank) {
        ArArgs b = a;
        b.resid = nullptr;
        ar_finish_row<AR_THREADS>(b, t, v, AR_MAXV, red);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned done = atomicAdd(a.counter + 4, 1u);
    if (done == gridDim.x - 1) {
      a.counter[4] = 0u;
      a.counter[2] += 2u * gridDim.x;
      a.counter[3] += 2u;
      *cm.epoch = epoch + 2u;
      __threadfence();
    }
  }
}

// ---- counted: latency-optimal for a few rows --------------------------------------------------------------------------------
// One CTA per row, plain launch, no grid barrier, no arrival counter: every rank adds its row into 64-bit slots on every
// GPU (top 8 bits count contributions, low 56 bits hold the biased fixed-point sum; multimem.red.add.u64 through
// NVSwitch or one red per peer), then polls ITS OWN copy of the slots until every word has counted all ranks, decodes,
// clears the word for its next use and finishes the row (residual, RMSNorm). One one-way trip through the switch;
// integer sums make every rank decode the same bits. Slot region: [4 call parities][IHB_ARC_MAX_ROWS * H] 64-bit words,
// which must start zeroed and must not be shared with the one-shot / two-shot regions. `x` may be fp32 or bf16.
constexpr unsigned long long ARC_ONE = 1ull << 56;
constexpr long long ARC_BIAS = 1ll << 51, ARC_QMAX = 1ll << 50;
constexpr float ARC_FIX = 268435456.f;                 // 2^28
constexpr int ARC_THREADS = 512, ARC_MAXV = 4;         // H <= 8192
struct ArcArgs {
  ArArgs a;
  int x_is_bf16;
  unsigned* call_counter;      // local, one word per row: calls made so far on this slot region (selects the parity)
};
__global__ void __launch_bounds__(ARC_THREADS) ar_counted_kernel(const ArcArgs q) {
  __shared__ float red[ARC_THREADS / 32];
  const ArArgs& a = q.a;
  const IhbComm& cm = a.comm;
  const int H = a.H, t = blockIdx.x, tid = threadIdx.x;
  pdl_wait();                                            // the previous call on this stream wrote the counter and cleared its words
  const unsigned call = q.call_counter[t];
  // a row's slots sit at a place that does not depend on T, and every row keeps its own call count: calls with
  // different numbers of rows can follow each other on the same region
  const size_t n = static_cast<size_t>(IHB_ARC_MAX_ROWS) * H;
  const size_t off0 = static_cast<size_t>(call & 3u) * n + static_cast<size_t>(t) * H;
  unsigned long long* local = reinterpret_cast<unsigned long long*>(cm.slots_local) + off0;
  const unsigned nr = static_cast<unsigned>(cm.nranks);
  for (int i = tid; i < H; i += ARC_THREADS) {
    const float v = q.x_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.x)[static_cast<size_t>(t) * H + i])
                                : a.x[static_cast<size_t>(t) * H + i];
    long long fx = __float2ll_rn(v * ARC_FIX);
    fx = fx > ARC_QMAX ? ARC_QMAX : (fx < -ARC_QMAX ? -ARC_QMAX : fx);
    const unsigned long long w = ARC_ONE + static_cast<unsigned long long>(fx + ARC_BIAS);
    if (nr == 1) {
      local[i] = w;
    } else if (cm.slots_mc != nullptr) {
      asm volatile("multimem.red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(reinterpret_cast<unsigned long long*>(cm.slots_mc) + off0 + i), "l"(w) : "memory");
    } else {
      for (int p = 0; p < cm.nranks; ++p)
        asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(reinterpret_cast<unsigned long long*>(cm.slots_peer[p]) + off0 + i), "l"(w) : "memory");
    }
  }
  __threadfence_block();
  float4 v[ARC_MAXV];
  bool ok = true;
  const unsigned long long t0 = globaltimer_ns();
  for (int j = 0; j < ARC_MAXV; ++j) {
    const int i = (tid + ARC_THREADS * j) * 4;
    v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i >= H) continue;
    unsigned long long w[4];
    unsigned spins = 0;
    for (;;) {
#pragma unroll
      for (int e = 0; e < 4; ++e) asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w[e]) : "l"(local + i + e) : "memory");
      if (!ok || ((w[0] >> 56) == nr && (w[1] >> 56) == nr && (w[2] >> 56) == nr && (w[3] >> 56) == nr)) break;
      if ((++spins & 63u) == 0u && (ld_cg_u(a.err) != 0u || globaltimer_ns() - t0 > IHB_PEER_WAIT_NS)) {
        set_error(a.err, ERR_PEER_BARRIER_TIMEOUT);
        ok = false;
      }
    }
    float f[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const long long sfx = static_cast<long long>(w[e] & (ARC_ONE - 1ull)) - static_cast<long long>(nr) * ARC_BIAS;
      f[e] = __ll2float_rn(sfx) * (1.f / ARC_FIX);
      local[i + e] = 0ull;                               // this thread is the word's only reader: clear it for its next use
    }
    v[j] = make_float4(f[0], f[1], f[2], f[3]);
  }
  pdl_launch_dependents();                               // the next kernel's launch overlaps the row's tail
  ar_finish_row<ARC_THREADS>(a, t, v, ARC_MAXV, red);
  for (int j = 0; j < ARC_MAXV; ++j) {
    const int i = (tid + ARC_THREADS * j) * 4;
    if (i < H) *reinterpret_cast<float4*>(a.out + static_cast<size_t>(t) * H + i) = v[j];
  }
  // every row keeps its own call count (read by the same row of the next launch): no cross-CTA bookkeeping
  if (tid == 0) q.call_counter[t] = call + 1u;
}

}  // namespace ihb

using namespace ihb;

// The latency-optimal variant for a few rows (see ar_counted_kernel). slots: 4 * IHB_ARC_MAX_ROWS * H 64-bit words of the
// symmetric buffer that start zeroed and are used by this variant only; call_counter: IHB_ARC_MAX_ROWS unsigned (one per
// row), zero before the first call; every rank must make the same sequence of calls (any T each); counter is unused.
// x: fp32, or bf16 when x_is_bf16. T <= IHB_ARC_MAX_ROWS, H % 4 == 0, H <= 8192. Launched with programmatic stream serialisation: back-to-back calls overlap the
// launch of one with the tail of the other.
extern "C" int ihb_allreduce_counted(const IhbComm* comm, const void* x, int x_is_bf16, const float* resid, const float* gamma,
                                     float eps, int T, int H, float* out, float* out_norm, void* out_norm_bf16,
                                     unsigned* counter, unsigned* call_counter, unsigned* err, cudaStream_t stream) {
  if (T < 1 || T > IHB_ARC_MAX_ROWS || H < 4 || (H % 4) || H > ARC_MAXV * ARC_THREADS * 4 || comm == nullptr ||
      call_counter == nullptr) return cudaErrorInvalidValue;
  (void)counter;
  ArcArgs q;
  q.a.comm = *comm; q.a.x = reinterpret_cast<const float*>(x); q.a.resid = resid; q.a.gamma = gamma; q.a.out = out;
  q.a.out_norm = out_norm; q.a.out_norm_bf16 = out_norm_bf16; q.a.eps = eps; q.a.T = T; q.a.H = H; q.a.counter = counter; q.a.err = err;
  q.x_is_bf16 = x_is_bf16;
  q.call_counter = call_counter;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(T); cfg.blockDim = dim3(ARC_THREADS); cfg.dynamicSmemBytes = 0; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, ar_counted_kernel, q);
}

// algo: 0 = choose by size, 1 = one-shot, 2 = two-shot. Slot region needed (floats): one-shot 2 * nranks * T * H,
// two-shot 2 * T * H. counter: 8 unsigned, zero before the first launch.
extern "C" int ihb_allreduce_norm(const IhbComm* comm, const float* x, const float* resid, const float* gamma, float eps,
                                  int T, int H, float* out, float* out_norm, void* out_norm_bf16, unsigned* counter,
                                  unsigned* err, int algo, int grid, cudaStream_t stream) {
  if (T < 1 || H < 4 || (H % 4) || H > AR_MAXV * AR_THREADS * 4 || comm == nullptr || counter == nullptr) return cudaErrorInvalidValue;
  ArArgs a;
  a.comm = *comm; a.x = x; a.resid = resid; a.gamma = gamma; a.out = out; a.out_norm = out_norm; a.out_norm_bf16 = out_norm_bf16;
  a.eps = eps;
  a.T = T; a.H = H; a.counter = counter; a.err = err;
  const size_t bytes = static_cast<size_t>(T) * H * 4;
  if (algo == 0) algo = bytes <= (256u << 10) ? 1 : 2;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (grid <= 0) grid = algo == 1 ? (T < 8 ? (T < 2 ? 4 : 8) : (T < sms ? T : sms)) : sms;
  if (grid > sms) grid = sms;                      // the CTAs wait on one another: all must be resident
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(AR_THREADS);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (algo == 1) return cudaLaunchKernelEx(&cfg, ar_oneshot_kernel, a);
  return cudaLaunchKernelEx(&cfg, ar_twoshot_kernel, a);
}
