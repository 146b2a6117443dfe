// Multi-token ("window") kernels around the tensor-core GEMMs: prompt chunks and speculative-verify windows.
//   * row-wise RMSNorm + per-token activation quantisation (e4m3 with one scale per 128 channels, or bf16) in the
//     layout the tcgen05 GEMM reads (X [T, K] row-major, scales [K / 128][T]);
//   * per-head QK RMSNorm + NeoX RoPE at explicit positions + KV-cache writes at explicit slots;
//   * window attention: T queries over the cached context plus the window's own rows, causal or with an explicit
//     visibility mask among the window tokens (token trees).
// The reference has these as SIMT prefill kernels (kernels/prefill_attn.cu:156-271: rmsnorm_rows, qknorm_rope,
// flash_attn_causal) and as the tree-verify attention of engine/native/mk_tree_attn*.cu.
#include "common.cuh"
#include "tails.cuh"

namespace ihb {

constexpr int WHD = 128;

// ---- RMSNorm (optional) + activation quantisation, one CTA (128 threads) per token ------------------------------------
// x [T][K] fp32 -> xn [T][K] fp32 (optional), xq [T][K] e4m3 / bf16, xs [K / 128][T]. gamma == NULL: no norm.
__global__ void __launch_bounds__(128) norm_quant_rows_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                              float eps, int K, int T, float* __restrict__ xn,
                                                              uint8_t* __restrict__ xq, float* __restrict__ xs, int fp8) {
  __shared__ float red[4];
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = x + static_cast<size_t>(t) * K;
  float rinv = 1.f;
  if (gamma != nullptr) {
    float ss = 0.f;
    for (int i = tid * 4; i < K; i += 512) {
      const float4 v = *reinterpret_cast<const float4*>(row + i);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    rinv = rsqrtf((red[0] + red[1] + red[2] + red[3]) / static_cast<float>(K) + eps);
  }
  // a warp handles one group of 128 channels at a time (the last group may be partial)
  for (int g0 = warp * 128; g0 < K; g0 += 512) {
    const int i = g0 + lane * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < K) {
      v = *reinterpret_cast<const float4*>(row + i);
      if (gamma != nullptr) {
        const float4 g = *reinterpret_cast<const float4*>(gamma + i);
        v = make_float4(v.x * rinv * g.x, v.y * rinv * g.y, v.z * rinv * g.z, v.w * rinv * g.w);
      }
      if (xn != nullptr) *reinterpret_cast<float4*>(xn + static_cast<size_t>(t) * K + i) = v;
    }
    if (fp8) {
      const float m = warp_max(fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
      const float sc = fmaxf(m, 1e-12f) * (1.f / 448.f);
      const float inv = 1.f / sc;
      const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v.x * inv, v.y * inv), __NV_SATFINITE, __NV_E4M3);
      const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v.z * inv, v.w * inv), __NV_SATFINITE, __NV_E4M3);
      if (i < K) *reinterpret_cast<uint32_t*>(xq + static_cast<size_t>(t) * K + i) = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
      if (lane == 0) xs[static_cast<size_t>(g0 >> 7) * T + t] = sc;
    } else if (i < K) {
      store_bf16x4(v, xq + (static_cast<size_t>(t) * K + i) * 2);
    }
  }
}

// ---- per-head QK RMSNorm + RoPE + KV append for T tokens: grid (nq + 2 nkv, T), one warp per head -------------------------
__global__ void __launch_bounds__(32) qk_norm_rope_rows_kernel(float* __restrict__ qkv, int nq, int nkv,
                                                               const float* __restrict__ q_gamma,
                                                               const float* __restrict__ k_gamma, float eps,
                                                               const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                               const int* __restrict__ positions, const int* __restrict__ slots,
                                                               __nv_bfloat16* __restrict__ k_cache,
                                                               __nv_bfloat16* __restrict__ v_cache, int max_seq) {
  const int head = blockIdx.x, t = blockIdx.y, lane = threadIdx.x;
  const int pos = min(positions[t], max_seq - 1), slot = min(slots[t], max_seq - 1);
  float* x = qkv + (static_cast<size_t>(t) * (nq + 2 * nkv) + head) * WHD;
  if (head >= nq + nkv) {
    __nv_bfloat16* dst = v_cache + (static_cast<size_t>(head - nq - nkv) * max_seq + slot) * WHD;
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[lane + 32 * j] = __float2bfloat16(x[lane + 32 * j]);
    return;
  }
  const float* gamma = head < nq ? q_gamma : k_gamma;
  float v[4], ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) { v[j] = x[lane + 32 * j]; ss += v[j] * v[j]; }
  ss = warp_sum(ss);
  const float rinv = rsqrtf(ss / static_cast<float>(WHD) + eps);
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = v[j] * rinv * gamma[lane + 32 * j];
  float o[4];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float c = cos_t[static_cast<size_t>(pos) * (WHD / 2) + lane + 32 * j];
    const float s = sin_t[static_cast<size_t>(pos) * (WHD / 2) + lane + 32 * j];
    o[j] = v[j] * c - v[j + 2] * s;
    o[j + 2] = v[j + 2] * c + v[j] * s;
  }
  if (head < nq) {
#pragma unroll
    for (int j = 0; j < 4; ++j) x[lane + 32 * j] = o[j];
  } else {
    __nv_bfloat16* dst = k_cache + (static_cast<size_t>(head - nq) * max_seq + slot) * WHD;
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[lane + 32 * j] = __float2bfloat16(o[j]);
  }
}

// ---- window attention: grid (T, nkv, q_per_kv / GQ), 128 threads (4 warps x 32 key positions per round) ----------------------
// Query t sees cache rows [0, base) and the window row base + j when mask[t][j] != 0 (mask == NULL: j <= t).
constexpr int WA_WARPS = 4;

template <int GQ>
__global__ void __launch_bounds__(WA_WARPS * 32) window_attn_kernel(
    const float* __restrict__ qkv, int qkv_stride, const __nv_bfloat16* __restrict__ k_cache,
    const __nv_bfloat16* __restrict__ v_cache, int nq, int nkv, int max_seq, int base, int T,
    const uint8_t* __restrict__ mask, float* __restrict__ out) {
  __shared__ __align__(16) float q_s[GQ][WHD];
  __shared__ __align__(16) float p_s[WA_WARPS][GQ][32];
  __shared__ float m_s[WA_WARPS][GQ], l_s[WA_WARPS][GQ];
  __shared__ __align__(16) float acc_s[WA_WARPS][GQ][WHD];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t = blockIdx.x, kvh = blockIdx.y, grp = blockIdx.z;
  const int q_per_kv = nq / nkv;
  const int gq = min(GQ, q_per_kv - grp * GQ);
  const int head0 = kvh * q_per_kv + grp * GQ;
  const int n = mask != nullptr ? base + T : base + t + 1;
  const float qscale = 0.08838834764831845f * 1.4426950408889634f;   // 1 / sqrt(128) * log2(e)
  for (int i = tid; i < GQ * WHD; i += WA_WARPS * 32) {
    const int g = i / WHD;
    q_s[g][i % WHD] = g < gq ? qkv[static_cast<size_t>(t) * qkv_stride + static_cast<size_t>(head0 + g) * WHD + (i % WHD)] * qscale : 0.f;
  }
  __syncthreads();
  float m[GQ], l[GQ], acc[GQ][4];
#pragma unroll
  for (int g = 0; g < GQ; ++g) { m[g] = -INFINITY; l[g] = 0.f; acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f; }
  const __nv_bfloat16* kbase = k_cache + static_cast<size_t>(kvh) * max_seq * WHD;
  const __nv_bfloat16* vbase = v_cache + static_cast<size_t>(kvh) * max_seq * WHD;
  for (int b0 = warp * 32; b0 < n; b0 += WA_WARPS * 32) {
    const int p = b0 + lane;
    bool valid = p < n;
    if (valid && p >= base && mask != nullptr) valid = mask[static_cast<size_t>(t) * T + (p - base)] != 0;
    if (__ballot_sync(0xffffffffu, valid) == 0u) continue;           // a fully masked round (token trees)
    float s[GQ];
#pragma unroll
    for (int g = 0; g < GQ; ++g) s[g] = 0.f;
    if (valid) {
      const uint4* kr = reinterpret_cast<const uint4*>(kbase + static_cast<size_t>(p) * WHD);
      uint4 kreg[WHD / 8];
#pragma unroll
      for (int c = 0; c < WHD / 8; ++c) kreg[c] = kr[c];
#pragma unroll
      for (int c = 0; c < WHD / 8; ++c) {
        const uint4 kv = kreg[c];
        float kf[8];
        kf[0] = __uint_as_float(kv.x << 16); kf[1] = __uint_as_float(kv.x & 0xffff0000u);
        kf[2] = __uint_as_float(kv.y << 16); kf[3] = __uint_as_float(kv.y & 0xffff0000u);
        kf[4] = __uint_as_float(kv.z << 16); kf[5] = __uint_as_float(kv.z & 0xffff0000u);
        kf[6] = __uint_as_float(kv.w << 16); kf[7] = __uint_as_float(kv.w & 0xffff0000u);
#pragma unroll
        for (int g = 0; g < GQ; ++g) {
          const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][c * 8]);
          const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][c * 8 + 4]);
          s[g] = fmaf(kf[0], qa.x, s[g]); s[g] = fmaf(kf[1], qa.y, s[g]);
          s[g] = fmaf(kf[2], qa.z, s[g]); s[g] = fmaf(kf[3], qa.w, s[g]);
          s[g] = fmaf(kf[4], qb.x, s[g]); s[g] = fmaf(kf[5], qb.y, s[g]);
          s[g] = fmaf(kf[6], qb.z, s[g]); s[g] = fmaf(kf[7], qb.w, s[g]);
        }
      }
    }
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
      const float sv = valid ? s[g] : -INFINITY;
      const float mnew = fmaxf(m[g], warp_max(sv));                  // finite: some lane of the round is valid
      const float corr = exp2f(m[g] - mnew);
      const float pv = valid ? exp2f(sv - mnew) : 0.f;
      m[g] = mnew;
      l[g] = l[g] * corr + pv;
      acc[g][0] *= corr; acc[g][1] *= corr; acc[g][2] *= corr; acc[g][3] *= corr;
      p_s[warp][g][lane] = pv;
    }
    __syncwarp();
    const int cnt = min(32, n - b0);
    for (int j0 = 0; j0 < cnt; j0 += 8) {
      uint2 vreg[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int jj = min(j0 + u, cnt - 1);                         // rows past the end repeat the last row; their p is 0
        vreg[u] = *reinterpret_cast<const uint2*>(vbase + static_cast<size_t>(b0 + jj) * WHD + lane * 4);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float v0 = __uint_as_float(vreg[u].x << 16), v1 = __uint_as_float(vreg[u].x & 0xffff0000u);
        const float v2 = __uint_as_float(vreg[u].y << 16), v3 = __uint_as_float(vreg[u].y & 0xffff0000u);
#pragma unroll
        for (int g = 0; g < GQ; ++g) {
          const float pj = (j0 + u < cnt) ? p_s[warp][g][j0 + u] : 0.f;
          acc[g][0] = fmaf(pj, v0, acc[g][0]); acc[g][1] = fmaf(pj, v1, acc[g][1]);
          acc[g][2] = fmaf(pj, v2, acc[g][2]); acc[g][3] = fmaf(pj, v3, acc[g][3]);
        }
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    const float lt = warp_sum(l[g]);
    if (lane == 0) { m_s[warp][g] = m[g]; l_s[warp][g] = lt; }
    *reinterpret_cast<float4*>(&acc_s[warp][g][lane * 4]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
  }
  __syncthreads();
  for (int i = tid; i < gq * WHD; i += WA_WARPS * 32) {
    const int g = i / WHD, d = i % WHD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WA_WARPS; ++w) M = fmaxf(M, m_s[w][g]);
    float a = 0.f, L = 0.f;
    if (M > -INFINITY) {
#pragma unroll
      for (int w = 0; w < WA_WARPS; ++w) {
        const float f = exp2f(m_s[w][g] - M);
        a += acc_s[w][g][d] * f;
        L += l_s[w][g] * f;
      }
    }
    out[static_cast<size_t>(t) * nq * WHD + static_cast<size_t>(head0 + g) * WHD + d] = L > 0.f ? a / L : 0.f;
  }
}

}  // namespace ihb

using namespace ihb;

extern "C" int ihb_norm_quant_rows(const float* x, const float* gamma, float eps, int K, int T, float* xn,
                                   unsigned char* xq, float* xs, int fp8, cudaStream_t stream) {
  if (T < 1 || K < 4 || (K % 4)) return cudaErrorInvalidValue;
  norm_quant_rows_kernel<<<T, 128, 0, stream>>>(x, gamma, eps, K, T, xn, xq, xs, fp8);
  return cudaGetLastError();
}

extern "C" int ihb_qk_norm_rope_rows(float* qkv, int nq, int nkv, const float* q_gamma, const float* k_gamma, float eps,
                                     const float* cos_t, const float* sin_t, const int* positions, const int* slots,
                                     void* k_cache, void* v_cache, int max_seq, int T, cudaStream_t stream) {
  if (T < 1) return cudaErrorInvalidValue;
  qk_norm_rope_rows_kernel<<<dim3(nq + 2 * nkv, T), 32, 0, stream>>>(
      qkv, nq, nkv, q_gamma, k_gamma, eps, cos_t, sin_t, positions, slots, reinterpret_cast<__nv_bfloat16*>(k_cache),
      reinterpret_cast<__nv_bfloat16*>(v_cache), max_seq);
  return cudaGetLastError();
}

extern "C" int ihb_window_attention(const float* qkv, int qkv_stride, const void* k_cache, const void* v_cache, int nq,
                                    int nkv, int max_seq, int base, int T, const unsigned char* mask, float* out,
                                    cudaStream_t stream) {
  if (T < 1 || nq % nkv || base + T > max_seq) return cudaErrorInvalidValue;
  const int q_per_kv = nq / nkv;
  const dim3 grid(T, nkv, (q_per_kv + 7) / 8);
  window_attn_kernel<8><<<grid, WA_WARPS * 32, 0, stream>>>(qkv, qkv_stride, reinterpret_cast<const __nv_bfloat16*>(k_cache),
                                                           reinterpret_cast<const __nv_bfloat16*>(v_cache), nq, nkv, max_seq,
                                                           base, T, mask, out);
  return cudaGetLastError();
}
