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
template <bool KV8>        // KV8: e4m3 cache rows with one fp32 scale per (KV head, slot), written here
__global__ void __launch_bounds__(32) qk_norm_rope_rows_kernel(float* __restrict__ qkv, int nq, int nkv,
                                                               const float* __restrict__ q_gamma,
                                                               const float* __restrict__ k_gamma, float eps,
                                                               const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                               const int* __restrict__ positions, const int* __restrict__ slots,
                                                               void* __restrict__ k_cache, void* __restrict__ v_cache,
                                                               float* __restrict__ k_scale, float* __restrict__ v_scale,
                                                               int max_seq) {
  const int head = blockIdx.x, t = blockIdx.y, lane = threadIdx.x;
  const int pos = min(positions[t], max_seq - 1), slot = min(slots[t], max_seq - 1);
  float* x = qkv + (static_cast<size_t>(t) * (nq + 2 * nkv) + head) * WHD;
  if (head >= nq + nkv) {
    float vv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) vv[j] = x[lane + 32 * j];
    kv_store_row<KV8>(v_cache, v_scale, static_cast<size_t>(head - nq - nkv) * max_seq + slot, vv, lane);
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
    kv_store_row<KV8>(k_cache, k_scale, static_cast<size_t>(head - nq) * max_seq + slot, o, lane);
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


// ---- window attention on the tensor cores: grid (ceil(T / 16), nkv, q_per_kv / 8), 8 warps -----------------------------------
// A CTA takes 16 consecutive window tokens and up to 8 query heads of one KV head: warp w owns head w, its 16 tokens
// are the 16 rows of m16n8k16 tiles. K / V blocks of 64 positions are staged once in shared memory for all heads
// (the per-token kernel above re-reads the whole context for every query token). Scores: q (bf16 head + bf16
// remainder, so that the product keeps fp32 accuracy against the bf16 cache rows) times K^T; online softmax in the
// log2 domain on the accumulator fragments; the probabilities (split the same way) go back in as the A operand of P V
// without leaving registers (the accumulator layout of two neighbouring 8-wide tiles is the A layout of one 16-deep step).
// Reference: kernels/prefill_attn.cu:212-271 (SIMT flash_attn_causal), engine/native/tc_verify_attn.cuh:48-119.
constexpr int WM_KB = 64;                 // key positions per block
constexpr int WM_REC = WHD + 4;           // partial record of a key slice: 128 channels, m, l, 2 pad (16-byte multiple)
constexpr int WM_LD = WHD + 8;            // padded row: fragment loads of a quarter warp cover all banks

__device__ __forceinline__ void wm_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned wm_pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}
// (x, y) -> bf16 heads packed, and the packed bf16 remainders
__device__ __forceinline__ void wm_split2(float x, float y, unsigned& hi, unsigned& lo) {
  const __nv_bfloat16 hx = __float2bfloat16(x), hy = __float2bfloat16(y);
  const __nv_bfloat162 h = __halves2bfloat162(hx, hy);
  hi = *reinterpret_cast<const unsigned*>(&h);
  lo = wm_pack_bf16(x - __bfloat162float(hx), y - __bfloat162float(hy));
}

// (x, y, z, w) * s -> four bf16 in two words
__device__ __forceinline__ uint2 wm_scaled_bf16x4(float4 v, float s) {
  return make_uint2(wm_pack_bf16(v.x * s, v.y * s), wm_pack_bf16(v.z * s, v.w * s));
}

template <int HPC, bool KV8>   // HPC: query heads (= warps) per CTA: 8, or 4 when 8 would leave most SMs without a CTA.
                               // KV8: e4m3 cache rows; a row is de-quantised (bytes * its scale -> bf16) on its way into
                               // shared memory, so the tensor-core loops below are the same for both cache types
__global__ void __launch_bounds__(HPC * 32) window_attn_mma_kernel(
    const float* __restrict__ qkv, int qkv_stride, const void* __restrict__ k_cache, const void* __restrict__ v_cache,
    const float* __restrict__ k_scale, const float* __restrict__ v_scale, int nq, int nkv, int max_seq, int base, int T,
    const uint8_t* __restrict__ mask, float* __restrict__ out, int nsplit, float* __restrict__ part) {
  __shared__ __align__(16) __nv_bfloat16 ks[WM_KB][WM_LD];
  __shared__ __align__(16) __nv_bfloat16 vs[WM_KB][WM_LD];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int split = blockIdx.x % nsplit;                // nsplit > 1: this CTA walks one slice of the key blocks
  const int t0 = (blockIdx.x / nsplit) * 16, kvh = blockIdx.y, grp = blockIdx.z;
  const int q_per_kv = nq / nkv;
  const int gq = min(HPC, q_per_kv - grp * HPC);
  const int head = kvh * q_per_kv + grp * HPC + warp;
  const bool active = warp < gq;
  const float qscale = 0.08838834764831845f * 1.4426950408889634f;   // 1 / sqrt(128) * log2(e)
  const int r0 = t0 + g, r1 = t0 + g + 8;                              // this thread's two rows (window tokens)
  // Q fragments of the whole head dimension: 8 steps of 16 channels, head and remainder
  unsigned qh[8][4], ql[8][4];
#pragma unroll
  for (int ksi = 0; ksi < 8; ++ksi) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int c = ksi * 16 + half * 8 + 2 * t4;
      float2 a = make_float2(0.f, 0.f), b = make_float2(0.f, 0.f);
      if (active && r0 < T) a = *reinterpret_cast<const float2*>(qkv + static_cast<size_t>(r0) * qkv_stride + static_cast<size_t>(head) * WHD + c);
      if (active && r1 < T) b = *reinterpret_cast<const float2*>(qkv + static_cast<size_t>(r1) * qkv_stride + static_cast<size_t>(head) * WHD + c);
      wm_split2(a.x * qscale, a.y * qscale, qh[ksi][2 * half], ql[ksi][2 * half]);
      wm_split2(b.x * qscale, b.y * qscale, qh[ksi][2 * half + 1], ql[ksi][2 * half + 1]);
    }
  }
  float o[16][4];
#pragma unroll
  for (int nd = 0; nd < 16; ++nd) o[nd][0] = o[nd][1] = o[nd][2] = o[nd][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int n_keys = mask != nullptr ? base + T : min(base + T, base + t0 + 16);
  const size_t row0 = static_cast<size_t>(kvh) * max_seq;
  const __nv_bfloat16* kbase = reinterpret_cast<const __nv_bfloat16*>(k_cache) + row0 * WHD;     // bf16 rows
  const __nv_bfloat16* vbase = reinterpret_cast<const __nv_bfloat16*>(v_cache) + row0 * WHD;
  const uint8_t* kbase8 = reinterpret_cast<const uint8_t*>(k_cache) + row0 * WHD;                // e4m3 rows
  const uint8_t* vbase8 = reinterpret_cast<const uint8_t*>(v_cache) + row0 * WHD;
  const int blocks_per_split = ((n_keys + WM_KB - 1) / WM_KB + nsplit - 1) / nsplit;
  const int key_end = min(n_keys, (split + 1) * blocks_per_split * WM_KB);
  for (int kb0 = split * blocks_per_split * WM_KB; kb0 < key_end; kb0 += WM_KB) {
    __syncthreads();                                   // the previous block's readers are done
    for (int i = tid; i < WM_KB * 16; i += HPC * 32) {
      const int r = i >> 4, ch = i & 15;
      const int p = min(kb0 + r, n_keys - 1);          // rows past the end repeat a valid row; they are masked below
      if constexpr (KV8) {
        const uint2 kq = *reinterpret_cast<const uint2*>(kbase8 + static_cast<size_t>(p) * WHD + ch * 8);
        const uint2 vq = *reinterpret_cast<const uint2*>(vbase8 + static_cast<size_t>(p) * WHD + ch * 8);
        const float ksc = k_scale[row0 + p], vsc = v_scale[row0 + p];
        const uint2 k0 = wm_scaled_bf16x4(e4m3x4_to_float4(kq.x), ksc), k1 = wm_scaled_bf16x4(e4m3x4_to_float4(kq.y), ksc);
        const uint2 v0 = wm_scaled_bf16x4(e4m3x4_to_float4(vq.x), vsc), v1 = wm_scaled_bf16x4(e4m3x4_to_float4(vq.y), vsc);
        *reinterpret_cast<uint4*>(&ks[r][ch * 8]) = make_uint4(k0.x, k0.y, k1.x, k1.y);
        *reinterpret_cast<uint4*>(&vs[r][ch * 8]) = make_uint4(v0.x, v0.y, v1.x, v1.y);
      } else {
        *reinterpret_cast<uint4*>(&ks[r][ch * 8]) = *reinterpret_cast<const uint4*>(kbase + static_cast<size_t>(p) * WHD + ch * 8);
        *reinterpret_cast<uint4*>(&vs[r][ch * 8]) = *reinterpret_cast<const uint4*>(vbase + static_cast<size_t>(p) * WHD + ch * 8);
      }
    }
    __syncthreads();
    if (!active) continue;
    // ---- scores of 64 keys: 8 tiles of 8 keys ----
    float sc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      float d[4] = {0.f, 0.f, 0.f, 0.f}, e[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ksi = 0; ksi < 8; ++ksi) {
        const unsigned b0 = *reinterpret_cast<const unsigned*>(&ks[nt * 8 + g][ksi * 16 + 2 * t4]);
        const unsigned b1 = *reinterpret_cast<const unsigned*>(&ks[nt * 8 + g][ksi * 16 + 8 + 2 * t4]);
        wm_mma(d, qh[ksi][0], qh[ksi][1], qh[ksi][2], qh[ksi][3], b0, b1);
        wm_mma(e, ql[ksi][0], ql[ksi][1], ql[ksi][2], ql[ksi][3], b0, b1);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int p = kb0 + nt * 8 + 2 * t4 + (j & 1);
        const int r = (j < 2) ? r0 : r1;
        bool vis = r < T && p < n_keys;
        if (vis && p >= base) vis = mask != nullptr ? (mask[static_cast<size_t>(r) * T + (p - base)] != 0) : (p - base <= r);
        sc[nt][j] = vis ? d[j] + e[j] : -INFINITY;
      }
    }
    // ---- online softmax (rows r0: elements 0, 1; r1: elements 2, 3 of every tile) ----
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      mx0 = fmaxf(mx0, fmaxf(sc[nt][0], sc[nt][1]));
      mx1 = fmaxf(mx1, fmaxf(sc[nt][2], sc[nt][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float c0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - mn0), c1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - mn1);
    m0 = mn0; m1 = mn1;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      sc[nt][0] = (sc[nt][0] == -INFINITY) ? 0.f : exp2f(sc[nt][0] - mn0);
      sc[nt][1] = (sc[nt][1] == -INFINITY) ? 0.f : exp2f(sc[nt][1] - mn0);
      sc[nt][2] = (sc[nt][2] == -INFINITY) ? 0.f : exp2f(sc[nt][2] - mn1);
      sc[nt][3] = (sc[nt][3] == -INFINITY) ? 0.f : exp2f(sc[nt][3] - mn1);
      s0 += sc[nt][0] + sc[nt][1];
      s1 += sc[nt][2] + sc[nt][3];
    }
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    l0 = l0 * c0 + s0;
    l1 = l1 * c1 + s1;
#pragma unroll
    for (int nd = 0; nd < 16; ++nd) { o[nd][0] *= c0; o[nd][1] *= c0; o[nd][2] *= c1; o[nd][3] *= c1; }
    // ---- O += P V: 4 steps of 16 keys; the probabilities go in as a bf16 head plus a bf16 remainder ----
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      unsigned ah[4], al[4];
      wm_split2(sc[2 * kk][0], sc[2 * kk][1], ah[0], al[0]);
      wm_split2(sc[2 * kk][2], sc[2 * kk][3], ah[1], al[1]);
      wm_split2(sc[2 * kk + 1][0], sc[2 * kk + 1][1], ah[2], al[2]);
      wm_split2(sc[2 * kk + 1][2], sc[2 * kk + 1][3], ah[3], al[3]);
#pragma unroll
      for (int nd = 0; nd < 16; ++nd) {
        unsigned b0, b1;
        asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                     : "=r"(b0), "=r"(b1) : "r"(smem_u32(&vs[kk * 16 + (lane & 15)][nd * 8])));
        wm_mma(o[nd], ah[0], ah[1], ah[2], ah[3], b0, b1);
        wm_mma(o[nd], al[0], al[1], al[2], al[3], b0, b1);
      }
    }
  }
  if (active && nsplit > 1) {
    // un-normalised partial of this slice: [token][head][split][128 channels, m, l]; window_attn_merge_kernel folds them
    float* p0 = part + ((static_cast<size_t>(r0) * nq + head) * nsplit + split) * WM_REC;
    float* p1 = part + ((static_cast<size_t>(r1) * nq + head) * nsplit + split) * WM_REC;
#pragma unroll
    for (int nd = 0; nd < 16; ++nd) {
      const int c = nd * 8 + 2 * t4;
      if (r0 < T) *reinterpret_cast<float2*>(p0 + c) = make_float2(o[nd][0], o[nd][1]);
      if (r1 < T) *reinterpret_cast<float2*>(p1 + c) = make_float2(o[nd][2], o[nd][3]);
    }
    if (t4 == 0) {
      if (r0 < T) *reinterpret_cast<float2*>(p0 + WHD) = make_float2(m0, l0);
      if (r1 < T) *reinterpret_cast<float2*>(p1 + WHD) = make_float2(m1, l1);
    }
  } else if (active) {
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
    for (int nd = 0; nd < 16; ++nd) {
      const int c = nd * 8 + 2 * t4;
      if (r0 < T) *reinterpret_cast<float2*>(out + static_cast<size_t>(r0) * nq * WHD + static_cast<size_t>(head) * WHD + c) = make_float2(o[nd][0] * i0, o[nd][1] * i0);
      if (r1 < T) *reinterpret_cast<float2*>(out + static_cast<size_t>(r1) * nq * WHD + static_cast<size_t>(head) * WHD + c) = make_float2(o[nd][2] * i1, o[nd][3] * i1);
    }
  }
}

// One warp per (token, head): folds the slices' partials (scores are in the log2 domain).
__global__ void __launch_bounds__(128) window_attn_merge_kernel(const float* __restrict__ part, int nq, int nsplit, int T,
                                                                float* __restrict__ out) {
  const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (w >= T * nq) return;
  const float* rec = part + static_cast<size_t>(w) * nsplit * WM_REC;
  float mx = -INFINITY;
  for (int s = 0; s < nsplit; ++s) mx = fmaxf(mx, rec[s * WM_REC + WHD]);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float l = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float m = rec[s * WM_REC + WHD];
    if (m == -INFINITY) continue;
    const float f = exp2f(m - mx);
    const float4 v = *reinterpret_cast<const float4*>(rec + s * WM_REC + lane * 4);
    acc.x += f * v.x; acc.y += f * v.y; acc.z += f * v.z; acc.w += f * v.w;
    l += f * rec[s * WM_REC + WHD + 1];
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  *reinterpret_cast<float4*>(out + static_cast<size_t>(w) * WHD + lane * 4) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
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
  qk_norm_rope_rows_kernel<false><<<dim3(nq + 2 * nkv, T), 32, 0, stream>>>(
      qkv, nq, nkv, q_gamma, k_gamma, eps, cos_t, sin_t, positions, slots, k_cache, v_cache, nullptr, nullptr, max_seq);
  return cudaGetLastError();
}

// e4m3 cache rows [nkv, max_seq, 128] bytes with scales [nkv, max_seq] fp32
extern "C" int ihb_qk_norm_rope_rows_kv8(float* qkv, int nq, int nkv, const float* q_gamma, const float* k_gamma, float eps,
                                         const float* cos_t, const float* sin_t, const int* positions, const int* slots,
                                         void* k_cache, void* v_cache, float* k_scale, float* v_scale, int max_seq, int T,
                                         cudaStream_t stream) {
  if (T < 1 || k_scale == nullptr || v_scale == nullptr) return cudaErrorInvalidValue;
  qk_norm_rope_rows_kernel<true><<<dim3(nq + 2 * nkv, T), 32, 0, stream>>>(
      qkv, nq, nkv, q_gamma, k_gamma, eps, cos_t, sin_t, positions, slots, k_cache, v_cache, k_scale, v_scale, max_seq);
  return cudaGetLastError();
}

// Key slices per query tile for a window of T tokens: enough CTAs to cover the GPU when the tiles alone do not, at
// most one slice per 64-key block and IHB_WINDOW_MAX_SPLITS.
static int window_split_bound(int nq, int nkv, int T) {          // slices wanted, before the cap by the number of key blocks
  const int q_per_kv = nq / nkv;
  const int ctas8 = ((T + 15) / 16) * nkv * ((q_per_kv + 7) / 8);
  const int ctas = (ctas8 >= 120 || q_per_kv <= 4) ? ctas8 : ((T + 15) / 16) * nkv * ((q_per_kv + 3) / 4);
  // one to two waves of tiles: a causal window gives the tiles 1 .. n key blocks, and the kernel lasts as long as the
  // longest tile; two slices per tile halve that (measured, 1024 tokens x 8 heads: 84 us unsliced)
  if (ctas >= 74) return ctas < 296 ? 2 : 1;
  const int s = (148 + ctas - 1) / ctas;
  return s > IHB_WINDOW_MAX_SPLITS ? IHB_WINDOW_MAX_SPLITS : s;
}

extern "C" int ihb_window_attention_splits(int nq, int nkv, int base, int T) {
  if (nq < 1 || nkv < 1 || nq % nkv || T < 1) return 1;
  const int blocks = (base + T + WM_KB - 1) / WM_KB;
  const int s = window_split_bound(nq, nkv, T);
  if (s == 2 && blocks < 8) return 1;               // short key ranges: the merge would cost more than the slices save
  return s > blocks ? blocks : s;
}

extern "C" size_t ihb_window_attention_scratch_floats(int nq, int nkv, int T) {
  if (nq < 1 || nkv < 1 || nq % nkv || T < 1) return 0;
  return static_cast<size_t>(T) * nq * window_split_bound(nq, nkv, T) * WM_REC;
}

template <bool KV8>
static int window_attention_tiles(const float* qkv, int qkv_stride, const void* k_cache, const void* v_cache,
                                  const float* k_scale, const float* v_scale, int nq, int nkv, int max_seq, int base, int T,
                                  const unsigned char* mask, float* out, float* scratch, cudaStream_t stream) {
  if (T < 1 || nq % nkv || base + T > max_seq || qkv_stride % 2) return cudaErrorInvalidValue;
  const int q_per_kv = nq / nkv;
  const int ctas8 = ((T + 15) / 16) * nkv * ((q_per_kv + 7) / 8);
  // few query tiles (verify windows, short prompts): slice the keys so that the whole GPU works on them
  const int nsplit = scratch != nullptr ? ihb_window_attention_splits(nq, nkv, base, T) : 1;
  if (ctas8 >= 120 || q_per_kv <= 4) {
    const dim3 grid(((T + 15) / 16) * nsplit, nkv, (q_per_kv + 7) / 8);
    window_attn_mma_kernel<8, KV8><<<grid, 256, 0, stream>>>(qkv, qkv_stride, k_cache, v_cache, k_scale, v_scale, nq, nkv,
                                                              max_seq, base, T, mask, out, nsplit, scratch);
  } else {
    const dim3 grid(((T + 15) / 16) * nsplit, nkv, (q_per_kv + 3) / 4);
    window_attn_mma_kernel<4, KV8><<<grid, 128, 0, stream>>>(qkv, qkv_stride, k_cache, v_cache, k_scale, v_scale, nq, nkv,
                                                              max_seq, base, T, mask, out, nsplit, scratch);
  }
  if (nsplit > 1) window_attn_merge_kernel<<<(T * nq + 3) / 4, 128, 0, stream>>>(scratch, nq, nsplit, T, out);
  return cudaGetLastError();
}

extern "C" int ihb_window_attention(const float* qkv, int qkv_stride, const void* k_cache, const void* v_cache, int nq,
                                    int nkv, int max_seq, int base, int T, const unsigned char* mask, float* out, int mode,
                                    float* scratch, cudaStream_t stream) {
  if (mode != 1)            // tensor-core tiles (the default); mode 1 keeps the per-token CUDA-core kernel
    return window_attention_tiles<false>(qkv, qkv_stride, k_cache, v_cache, nullptr, nullptr, nq, nkv, max_seq, base, T, mask,
                                         out, scratch, stream);
  if (T < 1 || nq % nkv || base + T > max_seq) return cudaErrorInvalidValue;
  const int q_per_kv = nq / nkv;
  const dim3 grid(T, nkv, (q_per_kv + 7) / 8);
  window_attn_kernel<8><<<grid, WA_WARPS * 32, 0, stream>>>(qkv, qkv_stride, reinterpret_cast<const __nv_bfloat16*>(k_cache),
                                                           reinterpret_cast<const __nv_bfloat16*>(v_cache), nq, nkv, max_seq,
                                                           base, T, mask, out);
  return cudaGetLastError();
}

// the tensor-core tiles over an e4m3 cache ([nkv, max_seq, 128] bytes, scales [nkv, max_seq] fp32)
extern "C" int ihb_window_attention_kv8(const float* qkv, int qkv_stride, const void* k_cache, const void* v_cache,
                                        const float* k_scale, const float* v_scale, int nq, int nkv, int max_seq, int base,
                                        int T, const unsigned char* mask, float* out, float* scratch, cudaStream_t stream) {
  if (k_scale == nullptr || v_scale == nullptr) return cudaErrorInvalidValue;
  return window_attention_tiles<true>(qkv, qkv_stride, k_cache, v_cache, k_scale, v_scale, nq, nkv, max_seq, base, T, mask, out,
                                      scratch, stream);
}
