// Routing of a window of tokens (prompt chunks, verify windows) without a trip to the host or a library sort:
//   * fused router: logits = h W_r^T in fp32 from bf16 router rows, softmax, top-k (ties -> lowest id), optional
//     renormalisation - one CTA per group of RT_TOK tokens;
//   * group table: the (token, slot) pairs are bucketed by expert (counting sort in one CTA) and cut into groups of at
//     most `nt` rows, the table the grouped tcgen05 GEMMs read;
//   * dispatch gather: activation rows in expert order;
//   * combine: the experts' outputs, weighted, summed in slot order (deterministic) and added to the residual.
// The reference does this per token at batch 1 (kernels/k4_router.cu) and, for prefill, with a per-expert loop driven
// from the host (kernels/prefill_moe.cu:61-170).
#include <algorithm>
#include "common.cuh"

namespace ihb {

constexpr int RT_TOK = 8;          // tokens per CTA of the router kernel
constexpr int RT_THREADS = 256;
constexpr int RT_KC = 512;         // channels staged per round

// One warp: softmax over the E logits of token t, top-k (ties -> lowest id), optional renormalisation.
__device__ __forceinline__ void router_topk_tail(const float* __restrict__ lg_row, int E, int top_k, int renorm, int lane, int t,
                                                 float* __restrict__ logits_out, int* __restrict__ ti, float* __restrict__ tw) {
  float v[8];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int e = lane + 32 * j;
    v[j] = e < E ? lg_row[e] : -INFINITY;
    mx = fmaxf(mx, v[j]);
    if (logits_out != nullptr && e < E) logits_out[static_cast<size_t>(t) * E + e] = v[j];
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) sum += (lane + 32 * j < E) ? __expf(v[j] - mx) : 0.f;
  sum = warp_sum(sum);
  float my_p = 0.f;
  int my_e = 0;
  for (int k = 0; k < top_k; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (v[j] > bv) { bv = v[j]; bi = lane + 32 * j; }
    const float mv = warp_max(bv);
    const int wi = __reduce_min_sync(0xffffffffu, bv == mv ? bi : 0x7fffffff);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (lane + 32 * j == wi) v[j] = -INFINITY;
    if (lane == k) { my_p = __expf(mv - mx) / sum; my_e = wi; }
  }
  float den = 1.f;
  if (renorm) den = warp_sum(lane < top_k ? my_p : 0.f);
  if (lane < top_k) {
    ti[static_cast<size_t>(t) * top_k + lane] = my_e;
    tw[static_cast<size_t>(t) * top_k + lane] = my_p / den;
  }
}

// ---- short windows (verify, a few prompt tokens): one warp per expert, then one warp per token -------------------------------------
// The tile kernels below put 8 or 16 tokens on ONE CTA, which then reads the whole router alone (66 us for 128 x 4096).
// Here the router rows are spread over E / 4 CTAs; the logits go through a caller-provided [T][E] buffer.
__global__ void __launch_bounds__(128) router_logits_wide_kernel(const float* __restrict__ h, const __nv_bfloat16* __restrict__ W,
                                                                 int T, int H, int E, float* __restrict__ logits) {
  const int e = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (e >= E) return;
  const uint4* wr = reinterpret_cast<const uint4*>(W + static_cast<size_t>(e) * H);
  for (int t = 0; t < T; ++t) {
    const float4* x = reinterpret_cast<const float4*>(h + static_cast<size_t>(t) * H);
    float acc = 0.f;
    for (int c8 = lane; c8 < H / 8; c8 += 32) acc += dot8_bf16(wr[c8], x[2 * c8], x[2 * c8 + 1]);   // the row stays in L1 after t = 0
    acc = warp_sum(acc);
    if (lane == 0) logits[static_cast<size_t>(t) * E + e] = acc;
  }
}
__global__ void __launch_bounds__(128) router_topk_from_logits_kernel(const float* __restrict__ logits, int T, int E, int top_k,
                                                                      int renorm, int* __restrict__ ti, float* __restrict__ tw) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t < T) router_topk_tail(logits + static_cast<size_t>(t) * E, E, top_k, renorm, lane, t, nullptr, ti, tw);
}

// logits [T][E] (optional), ti [T][k] int32, tw [T][k] fp32. E <= 256, k <= 8, H % RT_KC == 0 or any multiple of 8.
__global__ void __launch_bounds__(RT_THREADS) router_topk_rows_kernel(const float* __restrict__ h, const __nv_bfloat16* __restrict__ W,
                                                                       int T, int H, int E, int top_k, int renorm,
                                                                       float* __restrict__ logits_out, int* __restrict__ ti,
                                                                       float* __restrict__ tw) {
  __shared__ __align__(16) float xs[RT_TOK][RT_KC];
  __shared__ float lg[RT_TOK][256];
  const int tid = threadIdx.x, t0 = blockIdx.x * RT_TOK;
  // thread -> expert e (and e + 128 when E > 128 ... up to 256) x token half: 256 threads = 128 experts x 2 halves of 4 tokens
  const int e0 = tid & 127, half = tid >> 7;
  float acc[2][RT_TOK / 2];
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int t = 0; t < RT_TOK / 2; ++t) acc[j][t] = 0.f;
  for (int k0 = 0; k0 < H; k0 += RT_KC) {
    const int kc = min(RT_KC, H - k0);
    __syncthreads();
    for (int i = tid * 4; i < RT_TOK * RT_KC; i += RT_THREADS * 4) {
      const int t = i / RT_KC, c = i - t * RT_KC;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (t0 + t < T && c < kc) v = *reinterpret_cast<const float4*>(h + static_cast<size_t>(t0 + t) * H + k0 + c);
      *reinterpret_cast<float4*>(&xs[t][c]) = v;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int e = e0 + 128 * j;
      if (e < E) {
        const uint4* wr = reinterpret_cast<const uint4*>(W + static_cast<size_t>(e) * H + k0);
        for (int c8 = 0; c8 < kc / 8; ++c8) {
          const uint4 w = wr[c8];
#pragma unroll
          for (int t = 0; t < RT_TOK / 2; ++t) {
            const float4* x = reinterpret_cast<const float4*>(&xs[half * (RT_TOK / 2) + t][c8 * 8]);
            acc[j][t] += dot8_bf16(w, x[0], x[1]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int t = 0; t < RT_TOK / 2; ++t)
      if (e0 + 128 * j < E) lg[half * (RT_TOK / 2) + t][e0 + 128 * j] = acc[j][t];
  __syncthreads();
  // one warp per token: softmax + top-k
  const int warp = tid >> 5, lane = tid & 31;
  const int t = t0 + warp;
  if (warp < RT_TOK && t < T) router_topk_tail(lg[warp], E, top_k, renorm, lane, t, logits_out, ti, tw);
}

// ---- the same router on the tensor cores: 16 tokens per CTA, logits as m16n8k16 tiles ---------------------------------------------
// h stays fp32 in shared memory and is split into a bf16 head and a bf16 remainder when a fragment is built, so the
// logits keep fp32 accuracy against the bf16 router rows (a router decision must not depend on activation rounding).
// Chunks of 64 channels of h [16][64] and of the router [E][64] arrive by cp.async through a ring of NS buffers (4 when
// the router has at most 128 experts, else 2: a chunk is small, so the loop runs at the latency of a load unless
// several are in flight); warp w owns the expert tiles w, w + 8, ... (8 experts each).
constexpr int RM_TOK = 16, RM_KC = 64, RM_HLD = RM_KC + 4, RM_WLD = RM_KC + 8;
struct RmSmem {
  float h[4][RM_TOK][RM_HLD];
  __nv_bfloat16 w[2 * 256][RM_WLD];          // NS buffers of (512 / NS) rows
  float lg[RM_TOK][256];
  __nv_bfloat16 hh[RM_TOK][RM_WLD], hl[RM_TOK][RM_WLD];   // the current chunk of h as bf16 heads and remainders
};
__device__ __forceinline__ void rm_cp16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void rm_split2(float x, float y, unsigned& hi, unsigned& lo) {
  const __nv_bfloat16 hx = __float2bfloat16(x), hy = __float2bfloat16(y);
  const __nv_bfloat162 h = __halves2bfloat162(hx, hy);
  const __nv_bfloat162 l = __floats2bfloat162_rn(x - __bfloat162float(hx), y - __bfloat162float(hy));
  hi = *reinterpret_cast<const unsigned*>(&h);
  lo = *reinterpret_cast<const unsigned*>(&l);
}
template <int NS>
__global__ void __launch_bounds__(256) router_topk_rows_mma_kernel(const float* __restrict__ h, const __nv_bfloat16* __restrict__ W,
                                                                   int T, int H, int E, int top_k, int renorm,
                                                                   float* __restrict__ logits_out, int* __restrict__ ti,
                                                                   float* __restrict__ tw) {
  extern __shared__ __align__(16) uint8_t rm_raw[];
  RmSmem& sm = *reinterpret_cast<RmSmem*>(rm_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int t0 = blockIdx.x * RM_TOK;
  const int nchunks = H / RM_KC;
  // gridDim.y > 1: the experts are split over gridDim.y CTAs per token tile (the router is read by twice as many SMs);
  // the logits then go to global memory and router_topk_from_logits_kernel selects.
  const int E_all = E;
  const int e_first = blockIdx.y * (E_all / gridDim.y);
  E = E_all / gridDim.y;
  W += static_cast<size_t>(e_first) * H;
  auto issue = [&](int c, int buf) {
    const int k0 = c * RM_KC;
    for (int i = tid; i < RM_TOK * (RM_KC / 4); i += 256) {           // 16 tokens x 16 pieces of 4 floats
      const int r = i / (RM_KC / 4), p = i % (RM_KC / 4);
      rm_cp16(&sm.h[buf][r][p * 4], h + static_cast<size_t>(min(t0 + r, T - 1)) * H + k0 + p * 4);
    }
    for (int i = tid; i < E * (RM_KC / 8); i += 256) {                 // E rows x 8 pieces of 8 bf16
      const int r = i / (RM_KC / 8), p = i % (RM_KC / 8);
      rm_cp16(&sm.w[buf * (512 / NS) + r][p * 8], W + static_cast<size_t>(r) * H + k0 + p * 8);
    }
  };
  float acc[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  // one commit group per chunk position, empty past the end, so that "all but the newest NS - 1 groups" is always chunk c
#pragma unroll
  for (int c = 0; c < NS - 1; ++c) {
    if (c < nchunks) issue(c, c);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int c = 0; c < nchunks; ++c) {
    const int buf = c % NS;
    if (c + NS - 1 < nchunks) issue(c + NS - 1, (c + NS - 1) % NS);      // the buffer chunk c - 1 used: its readers passed the barrier below
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group %0;" ::"n"(NS - 1) : "memory");
    __syncthreads();
    // split the chunk of h once for all eight warps (each warp doing it for itself was most of the kernel's instructions)
    {
      const int r = tid >> 4, p = (tid & 15) * 4;
      const float4 v = *reinterpret_cast<const float4*>(&sm.h[buf][r][p]);
      unsigned h0, l0, h1, l1;
      rm_split2(v.x, v.y, h0, l0);
      rm_split2(v.z, v.w, h1, l1);
      *reinterpret_cast<uint2*>(&sm.hh[r][p]) = make_uint2(h0, h1);
      *reinterpret_cast<uint2*>(&sm.hl[r][p]) = make_uint2(l0, l1);
    }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < RM_KC / 16; ++ks) {
      const int k0 = ks * 16 + 2 * t4;
      unsigned ah[4], al[4];
      ah[0] = *reinterpret_cast<const unsigned*>(&sm.hh[g][k0]);     al[0] = *reinterpret_cast<const unsigned*>(&sm.hl[g][k0]);
      ah[1] = *reinterpret_cast<const unsigned*>(&sm.hh[g + 8][k0]); al[1] = *reinterpret_cast<const unsigned*>(&sm.hl[g + 8][k0]);
      ah[2] = *reinterpret_cast<const unsigned*>(&sm.hh[g][k0 + 8]); al[2] = *reinterpret_cast<const unsigned*>(&sm.hl[g][k0 + 8]);
      ah[3] = *reinterpret_cast<const unsigned*>(&sm.hh[g + 8][k0 + 8]); al[3] = *reinterpret_cast<const unsigned*>(&sm.hl[g + 8][k0 + 8]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = (warp + 8 * j) * 8 + g;
        if ((warp + 8 * j) * 8 < E) {
          const unsigned b0 = *reinterpret_cast<const unsigned*>(&sm.w[buf * (512 / NS) + e][k0]);
          const unsigned b1 = *reinterpret_cast<const unsigned*>(&sm.w[buf * (512 / NS) + e][k0 + 8]);
          asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                       : "+f"(acc[j][0]), "+f"(acc[j][1]), "+f"(acc[j][2]), "+f"(acc[j][3])
                       : "r"(ah[0]), "r"(ah[1]), "r"(ah[2]), "r"(ah[3]), "r"(b0), "r"(b1));
          asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                       : "+f"(acc[j][0]), "+f"(acc[j][1]), "+f"(acc[j][2]), "+f"(acc[j][3])
                       : "r"(al[0]), "r"(al[1]), "r"(al[2]), "r"(al[3]), "r"(b0), "r"(b1));
        }
      }
    }
    __syncthreads();                 // the buffer is refilled by the next iteration's issue
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = (warp + 8 * j) * 8 + 2 * t4;
    if ((warp + 8 * j) * 8 < E) {
      if (e < E) { sm.lg[g][e] = acc[j][0]; sm.lg[g + 8][e] = acc[j][2]; }
      if (e + 1 < E) { sm.lg[g][e + 1] = acc[j][1]; sm.lg[g + 8][e + 1] = acc[j][3]; }
    }
  }
  __syncthreads();
  if (gridDim.y > 1) {
    for (int i = tid; i < RM_TOK * E; i += 256) {
      const int r = i / E, e = i - r * E;
      if (t0 + r < T) logits_out[static_cast<size_t>(t0 + r) * E_all + e_first + e] = sm.lg[r][e];
    }
    return;
  }
  // softmax + top-k: a warp takes tokens warp and warp + 8
  for (int r = warp; r < RM_TOK; r += 8) {
    const int t = t0 + r;
    if (t >= T) continue;
    float v[8];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane + 32 * j;
      v[j] = e < E ? sm.lg[r][e] : -INFINITY;
      mx = fmaxf(mx, v[j]);
      if (logits_out != nullptr && e < E) logits_out[static_cast<size_t>(t) * E + e] = v[j];
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) sum += (lane + 32 * j < E) ? __expf(v[j] - mx) : 0.f;
    sum = warp_sum(sum);
    float my_p = 0.f;
    int my_e = 0;
    for (int k = 0; k < top_k; ++k) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (v[j] > bv) { bv = v[j]; bi = lane + 32 * j; }
      const float mv = warp_max(bv);
      const int wi = __reduce_min_sync(0xffffffffu, bv == mv ? bi : 0x7fffffff);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (lane + 32 * j == wi) v[j] = -INFINITY;
      if (lane == k) { my_p = __expf(mv - mx) / sum; my_e = wi; }
    }
    float den = 1.f;
    if (renorm) den = warp_sum(lane < top_k ? my_p : 0.f);
    if (lane < top_k) {
      ti[static_cast<size_t>(t) * top_k + lane] = my_e;
      tw[static_cast<size_t>(t) * top_k + lane] = my_p / den;
    }
  }
}

// ---- group table: one CTA ------------------------------------------------------------------------------------------------------
// ti [pairs] global expert ids (pairs = T * k; ids outside [expert0, expert0 + E_local) are dropped) -> order [pairs]
// (pair index at each sorted position), inv [pairs] (sorted position of each pair, -1 if dropped), groups [gmax][4] =
// {local expert, first sorted row, rows, 0}, n_groups [1]. Groups hold at most nt rows.
__global__ void __launch_bounds__(1024) moe_group_table_kernel(const int* __restrict__ ti, int pairs, int expert0, int E_local, int nt,
                                                               int* __restrict__ order, int* __restrict__ inv,
                                                               int* __restrict__ groups, int* __restrict__ n_groups, int gmax) {
  __shared__ int cnt[256], offs[256], fill[256], gfirst[257];
  const int tid = threadIdx.x;
  if (tid < 256) { cnt[tid] = 0; fill[tid] = 0; }
  __syncthreads();
  for (int i = tid; i < pairs; i += 1024) {
    const int e = ti[i] - expert0;
    if (e >= 0 && e < E_local) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int o = 0, g = 0;
    for (int e = 0; e < E_local; ++e) {
      offs[e] = o; gfirst[e] = g;
      o += cnt[e];
      g += (cnt[e] + nt - 1) / nt;
    }
    gfirst[E_local] = g;
    *n_groups = min(g, gmax);
  }
  __syncthreads();
  // rows inside an expert's bucket keep the order of their pair index: a thread takes a contiguous run of pairs and the
  // runs are served expert by expert with a prefix over threads would cost more than it gives; the bucket order only
  // has to be a permutation (every row is computed on its own), so slots are handed out with an atomic counter
  for (int i = tid; i < pairs; i += 1024) {
    const int e = ti[i] - expert0;
    if (e >= 0 && e < E_local) {
      const int p = offs[e] + atomicAdd(&fill[e], 1);
      order[p] = i;
      inv[i] = p;
    } else {
      inv[i] = -1;
    }
  }
  for (int e = tid; e < E_local; e += 1024) {
    const int ng = gfirst[e + 1] - gfirst[e];
    for (int j = 0; j < ng; ++j) {
      const int g = gfirst[e] + j;
      if (g < gmax) {
        groups[4 * g + 0] = e;
        groups[4 * g + 1] = offs[e] + j * nt;
        groups[4 * g + 2] = min(nt, cnt[e] - j * nt);
        groups[4 * g + 3] = 0;
      }
    }
  }
}

// ---- dispatch gather: out[p] = src[order[p] / k] (rows of `row_bytes` bytes, a multiple of 16), p < n_rows[0] ------------------
__global__ void __launch_bounds__(256) moe_gather_rows_kernel(const uint8_t* __restrict__ src, const int* __restrict__ order, int k,
                                                              int row_bytes, int pairs, uint8_t* __restrict__ out) {
  const int chunks = row_bytes / 16;
  for (int p = blockIdx.x; p < pairs; p += gridDim.x) {
    const int tok = order[p] / k;
    const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<size_t>(tok) * row_bytes);
    uint4* d = reinterpret_cast<uint4*>(out + static_cast<size_t>(p) * row_bytes);
    for (int c = threadIdx.x; c < chunks; c += 256) d[c] = s[c];
  }
}

// ---- combine: y[t] = (resid ? resid[t] : 0) + sum over slots (in slot order) of tw[t][slot] * yg[inv[t * k + slot]] ------------
__global__ void __launch_bounds__(256) moe_combine_rows_kernel(const float* __restrict__ yg, const int* __restrict__ inv,
                                                               const float* __restrict__ tw, int k, int H, int T,
                                                               const float* __restrict__ resid, float* __restrict__ y) {
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    for (int i = threadIdx.x * 4; i < H; i += 1024) {
      float4 acc = resid != nullptr ? *reinterpret_cast<const float4*>(resid + static_cast<size_t>(t) * H + i)
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < k; ++s) {
        const int p = inv[t * k + s];
        if (p >= 0) {
          const float w = tw[t * k + s];
          const float4 v = *reinterpret_cast<const float4*>(yg + static_cast<size_t>(p) * H + i);
          acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
        }
      }
      *reinterpret_cast<float4*>(y + static_cast<size_t>(t) * H + i) = acc;
    }
  }
}

// ---- block-scaled e4m3 -> bf16 (the window path multiplies bf16 copies of fp8 weights): 16 weights per thread --------------------
// W [nmat][rows][K] e4m3, scale [nmat][ceil(rows / rb)][nkb] (one fp32 per rb x kb block), out bf16 of W's shape. K % 16 == 0.
__global__ void __launch_bounds__(256) dequant_bf16_kernel(const uint8_t* __restrict__ W, const float* __restrict__ scale,
                                                           size_t nmat, int rows, int K, int rb, int kb, int nrb, int nkb,
                                                           __nv_bfloat16* __restrict__ out) {
  const size_t per_row = static_cast<size_t>(K) / 16;
  const size_t total = nmat * rows * per_row;
  for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * 256) {
    const size_t rowi = i / per_row;
    const int c16 = static_cast<int>(i - rowi * per_row);
    const size_t m = rowi / rows;
    const int r = static_cast<int>(rowi - m * rows);
    const uint4 w = *reinterpret_cast<const uint4*>(W + rowi * K + static_cast<size_t>(c16) * 16);
    // a 16-element piece may straddle two K blocks only if kb is not a multiple of 16, which the formats here never have
    const float sc = scale[(m * nrb + r / rb) * nkb + (c16 * 16) / kb];
    const unsigned wv[4] = {w.x, w.y, w.z, w.w};
    unsigned o[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 lo = __half22float2(cvt_e4m3x2(static_cast<unsigned short>(wv[q] & 0xffffu)));
      const float2 hi = __half22float2(cvt_e4m3x2(static_cast<unsigned short>(wv[q] >> 16)));
      const __nv_bfloat162 a = __floats2bfloat162_rn(lo.x * sc, lo.y * sc), b = __floats2bfloat162_rn(hi.x * sc, hi.y * sc);
      o[2 * q] = *reinterpret_cast<const unsigned*>(&a);
      o[2 * q + 1] = *reinterpret_cast<const unsigned*>(&b);
    }
    uint4* dst = reinterpret_cast<uint4*>(out + rowi * K + static_cast<size_t>(c16) * 16);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

}  // namespace ihb

using namespace ihb;

extern "C" int ihb_dequant_bf16(const void* W, const float* scale, long long nmat, int rows, int K, int rb, int kb, int nrb, int nkb,
                                void* out, cudaStream_t stream) {
  if (nmat < 1 || rows < 1 || K < 16 || K % 16 || rb < 1 || kb < 16 || kb % 16) return cudaErrorInvalidValue;
  const size_t total = static_cast<size_t>(nmat) * rows * (K / 16);
  const int grid = static_cast<int>(std::min<size_t>((total + 255) / 256, 148 * 16));
  dequant_bf16_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const uint8_t*>(W), scale, static_cast<size_t>(nmat), rows, K, rb, kb,
                                                nrb, nkb, reinterpret_cast<__nv_bfloat16*>(out));
  return cudaGetLastError();
}

extern "C" int ihb_clear_last_error(void) { return static_cast<int>(cudaGetLastError()); }

extern "C" int ihb_router_topk_rows(const float* h, const void* router_bf16, int T, int H, int E, int top_k, int renorm,
                                    float* logits, int* ti, float* tw, cudaStream_t stream) {
  if (T < 1 || E < 1 || E > 256 || top_k < 1 || top_k > 8 || top_k > E || H % 8) return cudaErrorInvalidValue;
  if (logits != nullptr && T <= 32) {        // short windows with a logits buffer: router rows spread over E / 4 CTAs
    router_logits_wide_kernel<<<(E + 3) / 4, 128, 0, stream>>>(h, reinterpret_cast<const __nv_bfloat16*>(router_bf16), T, H, E, logits);
    router_topk_from_logits_kernel<<<(T + 3) / 4, 128, 0, stream>>>(logits, T, E, top_k, renorm, ti, tw);
    return cudaGetLastError();
  }
  if (H % RM_KC == 0 && T >= 4) {            // tensor-core tiles; very short windows and odd widths take the plain kernel
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(router_topk_rows_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(sizeof(RmSmem)));
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(router_topk_rows_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(sizeof(RmSmem)));
      if (e != cudaSuccess) return e;
      attr_set = true;
    }
    if (logits != nullptr && T >= 256 && E % 16 == 0 && E <= 256) {
      // long windows: two CTAs per token tile, each half of the experts (4-deep ring: at most 128 rows per buffer)
      router_topk_rows_mma_kernel<4><<<dim3((T + RM_TOK - 1) / RM_TOK, 2), 256, sizeof(RmSmem), stream>>>(
          h, reinterpret_cast<const __nv_bfloat16*>(router_bf16), T, H, E, top_k, renorm, logits, ti, tw);
      router_topk_from_logits_kernel<<<(T + 3) / 4, 128, 0, stream>>>(logits, T, E, top_k, renorm, ti, tw);
      return cudaGetLastError();
    }
    if (E <= 128)
      router_topk_rows_mma_kernel<4><<<(T + RM_TOK - 1) / RM_TOK, 256, sizeof(RmSmem), stream>>>(
          h, reinterpret_cast<const __nv_bfloat16*>(router_bf16), T, H, E, top_k, renorm, logits, ti, tw);
    else
      router_topk_rows_mma_kernel<2><<<(T + RM_TOK - 1) / RM_TOK, 256, sizeof(RmSmem), stream>>>(
          h, reinterpret_cast<const __nv_bfloat16*>(router_bf16), T, H, E, top_k, renorm, logits, ti, tw);
    return cudaGetLastError();
  }
  router_topk_rows_kernel<<<(T + RT_TOK - 1) / RT_TOK, RT_THREADS, 0, stream>>>(
      h, reinterpret_cast<const __nv_bfloat16*>(router_bf16), T, H, E, top_k, renorm, logits, ti, tw);
  return cudaGetLastError();
}

extern "C" int ihb_moe_group_table(const int* ti, int pairs, int expert0, int E_local, int nt, int* order, int* inv, int* groups,
                                   int* n_groups, int gmax, cudaStream_t stream) {
  if (pairs < 1 || E_local < 1 || E_local > 256 || nt < 1 || gmax < 1) return cudaErrorInvalidValue;
  moe_group_table_kernel<<<1, 1024, 0, stream>>>(ti, pairs, expert0, E_local, nt, order, inv, groups, n_groups, gmax);
  return cudaGetLastError();
}

extern "C" int ihb_moe_gather_rows(const void* src, const int* order, int k, int row_bytes, int pairs, void* out, cudaStream_t stream) {
  if (pairs < 1 || k < 1 || row_bytes % 16) return cudaErrorInvalidValue;
  moe_gather_rows_kernel<<<min(pairs, 148 * 8), 256, 0, stream>>>(reinterpret_cast<const uint8_t*>(src), order, k, row_bytes, pairs,
                                                                  reinterpret_cast<uint8_t*>(out));
  return cudaGetLastError();
}

extern "C" int ihb_moe_combine_rows(const float* yg, const int* inv, const float* tw, int k, int H, int T, const float* resid,
                                    float* y, cudaStream_t stream) {
  if (T < 1 || k < 1 || H % 4) return cudaErrorInvalidValue;
  moe_combine_rows_kernel<<<min(T, 148 * 8), 256, 0, stream>>>(yg, inv, tw, k, H, T, resid, y);
  return cudaGetLastError();
}
