// Routing of a window of tokens (prompt chunks, verify windows) without a trip to the host or a library sort:
//   * fused router: logits = h W_r^T in fp32 from bf16 router rows, softmax, top-k (ties -> lowest id), optional
//     renormalisation - one CTA per group of RT_TOK tokens;
//   * group table: the (token, slot) pairs are bucketed by expert (counting sort in one CTA) and cut into groups of at
//     most `nt` rows, the table the grouped tcgen05 GEMMs read;
//   * dispatch gather: activation rows in expert order;
//   * combine: the experts' outputs, weighted, summed in slot order (deterministic) and added to the residual.
// The reference does this per token at batch 1 (kernels/k4_router.cu) and, for prefill, with a per-expert loop driven
// from the host (kernels/prefill_moe.cu:61-170).
#include "common.cuh"

namespace ihb {

constexpr int RT_TOK = 8;          // tokens per CTA of the router kernel
constexpr int RT_THREADS = 256;
constexpr int RT_KC = 512;         // channels staged per round

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
  if (warp < RT_TOK && t < T) {
    float v[8];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane + 32 * j;
      v[j] = e < E ? lg[warp][e] : -INFINITY;
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

}  // namespace ihb

using namespace ihb;

extern "C" int ihb_router_topk_rows(const float* h, const void* router_bf16, int T, int H, int E, int top_k, int renorm,
                                    float* logits, int* ti, float* tw, cudaStream_t stream) {
  if (T < 1 || E < 1 || E > 256 || top_k < 1 || top_k > 8 || top_k > E || H % 8) return cudaErrorInvalidValue;
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
