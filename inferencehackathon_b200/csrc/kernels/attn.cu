// Decode-side attention kernels, head_dim = 128, sm_100a:
//   embed_norm          token embedding gather + first RMSNorm
//   qk_norm_rope_kv     per-head RMSNorm of Q and K, NeoX RoPE, KV-cache append (bf16)
//   flash_decode        split-KV GQA single-query attention; the last CTA of each head group merges the split
//                       partials in the same launch (the reference needs a second kernel,
//                       kernels/k2_flash_decode.cu:90-195) and every K/V row is read once for all query heads of
//                       its group (the reference re-reads it per 4 heads, kernels/decode_step_tp8.cu:1798-1802).
// The position counter lives in device memory so that a captured CUDA graph replays without host updates.
#include "common.cuh"
#include "api.h"
#include "tails.cuh"

namespace ihb {

constexpr int HD = 128;

// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) embed_norm_kernel(const void* __restrict__ embed, int is_bf16,
                                                         const int* __restrict__ token, int H,
                                                         const float* __restrict__ gamma, float eps,
                                                         float* __restrict__ resid, float* __restrict__ xn,
                                                         uint8_t* __restrict__ xq, float* __restrict__ xs, int xq_fp8) {
  __shared__ float red[8];
  pdl_wait();
  pdl_launch_dependents();
  const int tok = ld_cg_i(token);
  const int tid = threadIdx.x;
  constexpr int MAXV = 8;                  // H <= 8192, multiple of 4: float4 j of thread t covers (t + 256 j) * 4
  float4 v[MAXV];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = (tid + 256 * j) * 4;
    v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < H) {
      if (is_bf16) {
        const uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(embed) +
                                                        static_cast<size_t>(tok) * H + i);
        v[j] = make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u),
                           __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xffff0000u));
      } else {
        v[j] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(embed) + static_cast<size_t>(tok) * H + i);
      }
    }
    ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += red[w];
  const float rinv = rsqrtf(tot / static_cast<float>(H) + eps);
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = (tid + 256 * j) * 4;
    if (i < H) {
      const float4 g = *reinterpret_cast<const float4*>(gamma + i);
      const float4 o = make_float4(v[j].x * rinv * g.x, v[j].y * rinv * g.y, v[j].z * rinv * g.z, v[j].w * rinv * g.w);
      *reinterpret_cast<float4*>(resid + i) = v[j];
      *reinterpret_cast<float4*>(xn + i) = o;
      if (xq != nullptr) {                 // needs H % 128 == 0: a warp covers one group of 128 channels
        if (xq_fp8) quant_group128(o, xq + i, xs + (i >> 7), tid & 31);
        else store_bf16x4(o, xq + 2 * i);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// One warp per head. Lane owns channels d = lane + 32 j (j = 0..3); RoPE pairs (d, d + 64) are (j, j + 2).
// KV8: the cache rows are e4m3 with one fp32 scale per (KV head, position) = amax of the row / 448, written here;
// otherwise bf16 rows and the scale pointers are unused.
template <bool KV8>
__global__ void __launch_bounds__(32) qk_norm_rope_kv_kernel(float* __restrict__ qkv, int nq, int nkv,
                                                             const float* __restrict__ q_gamma,
                                                             const float* __restrict__ k_gamma, float eps,
                                                             const float* __restrict__ cos_t,
                                                             const float* __restrict__ sin_t,
                                                             const int* __restrict__ pos_p,
                                                             void* __restrict__ k_cache, void* __restrict__ v_cache,
                                                             float* __restrict__ k_scale, float* __restrict__ v_scale,
                                                             int max_seq) {
  pdl_wait();
  pdl_launch_dependents();
  const int head = blockIdx.x;
  const int lane = threadIdx.x;
  int pos = ld_cg_i(pos_p);
  if (pos >= max_seq) pos = max_seq - 1;   // cache full: keep overwriting the last row instead of running past it
  if (head >= nq + nkv) {                  // V head: copy into the cache
    const int kvh = head - nq - nkv;
    const float* v = qkv + static_cast<size_t>(head) * HD;
    float vv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) vv[j] = ld_cg_f(v + lane + 32 * j);
    kv_store_row<KV8>(v_cache, v_scale, static_cast<size_t>(kvh) * max_seq + pos, vv, lane);
    return;
  }
  float* x = qkv + static_cast<size_t>(head) * HD;
  const float* gamma = head < nq ? q_gamma : k_gamma;
  float v[4];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[j] = ld_cg_f(x + lane + 32 * j);
    ss += v[j] * v[j];
  }
  ss = warp_sum(ss);
  const float rinv = rsqrtf(ss / static_cast<float>(HD) + eps);
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = v[j] * rinv * gamma[lane + 32 * j];
  float o[4];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float c = cos_t[static_cast<size_t>(pos) * (HD / 2) + lane + 32 * j];
    const float s = sin_t[static_cast<size_t>(pos) * (HD / 2) + lane + 32 * j];
    o[j] = v[j] * c - v[j + 2] * s;
    o[j + 2] = v[j + 2] * c + v[j] * s;
  }
  if (head < nq) {
#pragma unroll
    for (int j = 0; j < 4; ++j) x[lane + 32 * j] = o[j];
  } else {
    kv_store_row<KV8>(k_cache, k_scale, static_cast<size_t>(head - nq) * max_seq + pos, o, lane);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// flash decode. grid = (nsplit, nkv, q_per_kv / GQ); block = 128 threads (4 warps x 32 positions).
// scratch layout per (head, split): [128 acc][m][l]  (FD_REC floats)
// ---------------------------------------------------------------------------------------------------------------------
constexpr int FD_WARPS = 4;
constexpr int FD_BLOCK = FD_WARPS * 32;     // positions per CTA iteration
constexpr int FD_REC = HD + 2;

template <int GQ, bool KV8>   // KV8: e4m3 cache rows with a scale per (KV head, position); the scores take the K scale, the
                              // probabilities the V scale, so the inner loops stay plain FMAs on decoded bytes
__global__ void __launch_bounds__(FD_WARPS * 32) flash_decode_kernel(
    const float* __restrict__ q, const void* __restrict__ k_cache, const void* __restrict__ v_cache,
    const float* __restrict__ k_scale, const float* __restrict__ v_scale, int nq, int nkv, int max_seq,
    const int* __restrict__ pos_p,
    int nsplit, float* __restrict__ scratch, unsigned* __restrict__ counters, float* __restrict__ out,
    uint8_t* __restrict__ out_q, float* __restrict__ out_s, int out_fp8) {
  __shared__ float red_m[FD_WARPS];
  __shared__ __align__(16) float q_s[GQ][HD];
  __shared__ __align__(16) float p_s[FD_WARPS][GQ][32];
  __shared__ float m_s[FD_WARPS][GQ], l_s[FD_WARPS][GQ];
  __shared__ __align__(16) float acc_s[FD_WARPS][GQ][HD];
  __shared__ int s_last;
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, grp = blockIdx.z;
  const int q_per_kv = nq / nkv;
  const int head0 = kvh * q_per_kv + grp * GQ;
  int n = ld_cg_i(pos_p) + 1;
  if (n > max_seq) n = max_seq;
  const float qscale = 0.08838834764831845f * 1.4426950408889634f;   // 1/sqrt(128) * log2(e)
  for (int i = tid; i < GQ * HD; i += FD_WARPS * 32)
    q_s[i / HD][i % HD] = ld_cg_f(q + static_cast<size_t>(head0) * HD + i) * qscale;
  __syncthreads();

  float m[GQ], l[GQ], acc[GQ][4];
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
    acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
  }
  const size_t row0 = static_cast<size_t>(kvh) * max_seq;
  const __nv_bfloat16* kbase = reinterpret_cast<const __nv_bfloat16*>(k_cache) + row0 * HD;      // bf16 rows
  const __nv_bfloat16* vbase = reinterpret_cast<const __nv_bfloat16*>(v_cache) + row0 * HD;
  const uint8_t* kbase8 = reinterpret_cast<const uint8_t*>(k_cache) + row0 * HD;                 // e4m3 rows
  const uint8_t* vbase8 = reinterpret_cast<const uint8_t*>(v_cache) + row0 * HD;

  for (int b0 = split * FD_BLOCK; b0 < n; b0 += nsplit * FD_BLOCK) {
    const int base = b0 + warp * 32;
    if (base >= n) break;
    const int p = base + lane;
    const bool valid = p < n;
    float s[GQ];
#pragma unroll
    for (int g = 0; g < GQ; ++g) s[g] = 0.f;
    float vsc = 0.f;                                   // V scale of this lane's position (KV8)
    if constexpr (KV8) {
      if (valid) {
        const uint4* kr = reinterpret_cast<const uint4*>(kbase8 + static_cast<size_t>(p) * HD);
        uint4 kreg[HD / 16];
#pragma unroll
        for (int c = 0; c < HD / 16; ++c) kreg[c] = kr[c];      // the row's 128 bytes in flight before the first FMA
        const float ksc = k_scale[row0 + p];
        vsc = v_scale[row0 + p];
#pragma unroll
        for (int c = 0; c < HD / 16; ++c) {
          const unsigned w4[4] = {kreg[c].x, kreg[c].y, kreg[c].z, kreg[c].w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float4 kf = e4m3x4_to_float4(w4[u]);
#pragma unroll
            for (int g = 0; g < GQ; ++g) {
              const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][c * 16 + u * 4]);
              s[g] = fmaf(kf.x, qa.x, s[g]); s[g] = fmaf(kf.y, qa.y, s[g]);
              s[g] = fmaf(kf.z, qa.z, s[g]); s[g] = fmaf(kf.w, qa.w, s[g]);
            }
          }
        }
#pragma unroll
        for (int g = 0; g < GQ; ++g) s[g] *= ksc;
      }
    } else if (valid) {
      const uint4* kr = reinterpret_cast<const uint4*>(kbase + static_cast<size_t>(p) * HD);
      uint4 kreg[HD / 8];
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) kreg[c] = kr[c];      // all 16 loads in flight before the first FMA
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
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
      const float mnew = fmaxf(m[g], warp_max(sv));     // finite: lane 0 of the chunk is always valid
      const float corr = exp2f(m[g] - mnew);
      const float pv = valid ? exp2f(sv - mnew) : 0.f;
      m[g] = mnew;
      l[g] = l[g] * corr + pv;                           // per-lane partial sum, combined at the end
      acc[g][0] *= corr; acc[g][1] *= corr; acc[g][2] *= corr; acc[g][3] *= corr;
      p_s[warp][g][lane] = KV8 ? pv * vsc : pv;          // the denominator keeps the unscaled probability
    }
    __syncwarp();
    const int cnt = min(32, n - base);
    if constexpr (KV8) {
      for (int j0 = 0; j0 < cnt; j0 += 8) {
        unsigned vreg[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int jj = min(j0 + u, cnt - 1);             // rows past the end repeat the last row; their p is 0
          vreg[u] = *reinterpret_cast<const unsigned*>(vbase8 + static_cast<size_t>(base + jj) * HD + lane * 4);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float4 vf = e4m3x4_to_float4(vreg[u]);
#pragma unroll
          for (int g = 0; g < GQ; ++g) {
            const float pj = p_s[warp][g][j0 + u];
            acc[g][0] = fmaf(pj, vf.x, acc[g][0]); acc[g][1] = fmaf(pj, vf.y, acc[g][1]);
            acc[g][2] = fmaf(pj, vf.z, acc[g][2]); acc[g][3] = fmaf(pj, vf.w, acc[g][3]);
          }
        }
      }
    } else {
      for (int j0 = 0; j0 < cnt; j0 += 8) {
        uint2 vreg[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int jj = min(j0 + u, cnt - 1);               // rows past the end repeat the last row; their p is 0
          vreg[u] = *reinterpret_cast<const uint2*>(vbase + static_cast<size_t>(base + jj) * HD + lane * 4);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float v0 = __uint_as_float(vreg[u].x << 16), v1 = __uint_as_float(vreg[u].x & 0xffff0000u);
          const float v2 = __uint_as_float(vreg[u].y << 16), v3 = __uint_as_float(vreg[u].y & 0xffff0000u);
#pragma unroll
          for (int g = 0; g < GQ; ++g) {
            const float pj = p_s[warp][g][j0 + u];
            acc[g][0] = fmaf(pj, v0, acc[g][0]); acc[g][1] = fmaf(pj, v1, acc[g][1]);
            acc[g][2] = fmaf(pj, v2, acc[g][2]); acc[g][3] = fmaf(pj, v3, acc[g][3]);
          }
        }
      }
    }
    __syncwarp();
  }

  // combine the four warps of the CTA
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    const float lt = warp_sum(l[g]);
    if (lane == 0) { m_s[warp][g] = m[g]; l_s[warp][g] = lt; }
    *reinterpret_cast<float4*>(&acc_s[warp][g][lane * 4]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
  }
  __syncthreads();
  for (int i = tid; i < GQ * HD; i += FD_WARPS * 32) {
    const int g = i / HD, d = i % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < FD_WARPS; ++w) M = fmaxf(M, m_s[w][g]);
    float a = 0.f, L = 0.f;
    if (M > -INFINITY) {
#pragma unroll
      for (int w = 0; w < FD_WARPS; ++w) {
        const float f = exp2f(m_s[w][g] - M);     // exp2(-inf) = 0 for warps without positions
        a += acc_s[w][g][d] * f;
        L += l_s[w][g] * f;
      }
    }
    float* rec = scratch + (static_cast<size_t>(head0 + g) * nsplit + split) * FD_REC;
    rec[d] = a;
    if (d == 0) { rec[HD] = M; rec[HD + 1] = L; }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    unsigned* ctr = counters + kvh * gridDim.z + grp;
    const unsigned old = atomicAdd(ctr, 1u);
    s_last = (old == static_cast<unsigned>(nsplit) - 1u);
    if (s_last) { *ctr = 0u; __threadfence(); }
  }
  __syncthreads();
  if (!s_last) return;
  // merge of the split partials by the last CTA of this (kv head, group). All loads of a phase are independent
  // (the loops over heads are unrolled), so the merge costs two memory round trips, not two per head.
  const int d = tid;                                   // 128 threads = 128 channels
  float* ml_s = &acc_s[0][0][0];                       // reuse: [GQ][nsplit] m, then [GQ][nsplit] l (nsplit <= 256)
  const int nml = GQ * nsplit;
  for (int i = tid; i < nml; i += FD_WARPS * 32) {
    const float* rec = scratch + (static_cast<size_t>(head0 + i / nsplit) * nsplit + (i % nsplit)) * FD_REC;
    ml_s[i] = ld_cg_f(rec + HD);
    ml_s[nml + i] = ld_cg_f(rec + HD + 1);
  }
  __syncthreads();
  float o[GQ];
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    const float* recs = scratch + static_cast<size_t>(head0 + g) * nsplit * FD_REC;
    float M = -INFINITY;
    for (int sp = 0; sp < nsplit; ++sp) M = fmaxf(M, ml_s[g * nsplit + sp]);
    float a = 0.f, L = 0.f;
#pragma unroll 4
    for (int sp = 0; sp < nsplit; ++sp) {
      const float ms = ml_s[g * nsplit + sp];
      const float f = (ms > -INFINITY) ? exp2f(ms - M) : 0.f;
      a = fmaf(ld_cg_f(recs + sp * FD_REC + d), f, a);     // empty splits wrote zeros
      L = fmaf(ml_s[nml + g * nsplit + sp], f, L);
    }
    o[g] = a / L;
  }
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    out[static_cast<size_t>(head0 + g) * HD + d] = o[g];
    if (out_q != nullptr) {
      // a head is one group of 128 channels of the o_proj input row
      if (out_fp8) {
        const float mx = warp_max(fabsf(o[g]));
        __syncthreads();
        if (lane == 0) red_m[warp] = mx;
        __syncthreads();
        const float amax = fmaxf(fmaxf(red_m[0], red_m[1]), fmaxf(red_m[2], red_m[3]));
        const float sc = fmaxf(amax, 1e-12f) * (1.f / 448.f);
        out_q[static_cast<size_t>(head0 + g) * HD + d] =
            static_cast<uint8_t>(__nv_cvt_float_to_fp8(o[g] / sc, __NV_SATFINITE, __NV_E4M3));
        if (tid == 0) out_s[head0 + g] = sc;
      } else {
        reinterpret_cast<__nv_bfloat16*>(out_q)[static_cast<size_t>(head0 + g) * HD + d] = __float2bfloat16(o[g]);
      }
    }
  }
}

static void pdl_cfg(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, dim3 grid, dim3 block, int use_pdl,
                    cudaStream_t stream) {
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl ? 1 : 0;
}

}  // namespace ihb

using namespace ihb;

extern "C" int ihb_embed_norm(const void* embed, int embed_is_bf16, const int* token, int H, const float* gamma,
                              float eps, float* resid, float* xn, unsigned char* xq, float* xs, int xq_fp8, int use_pdl,
                              cudaStream_t stream) {
  if (H % 4 || H > 8192 || (xq != nullptr && H % 128)) return cudaErrorInvalidValue;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  pdl_cfg(cfg, attr, dim3(1), dim3(256), use_pdl, stream);
  return cudaLaunchKernelEx(&cfg, embed_norm_kernel, embed, embed_is_bf16, token, H, gamma, eps, resid, xn, xq, xs, xq_fp8);
}

static int qk_norm_rope_kv_launch(float* qkv, int nq, int nkv, const float* q_gamma, const float* k_gamma, float eps,
                                  const float* cos_t, const float* sin_t, const int* pos, void* k_cache, void* v_cache,
                                  float* k_scale, float* v_scale, int max_seq, int use_pdl, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  pdl_cfg(cfg, attr, dim3(nq + 2 * nkv), dim3(32), use_pdl, stream);
  if (k_scale != nullptr)
    return cudaLaunchKernelEx(&cfg, qk_norm_rope_kv_kernel<true>, qkv, nq, nkv, q_gamma, k_gamma, eps, cos_t, sin_t, pos,
                              k_cache, v_cache, k_scale, v_scale, max_seq);
  return cudaLaunchKernelEx(&cfg, qk_norm_rope_kv_kernel<false>, qkv, nq, nkv, q_gamma, k_gamma, eps, cos_t, sin_t, pos,
                            k_cache, v_cache, k_scale, v_scale, max_seq);
}

extern "C" int ihb_qk_norm_rope_kv(float* qkv, int nq, int nkv, const float* q_gamma, const float* k_gamma,
                                   float eps, const float* cos_t, const float* sin_t, const int* pos, void* k_cache,
                                   void* v_cache, int max_seq, int use_pdl, cudaStream_t stream) {
  return qk_norm_rope_kv_launch(qkv, nq, nkv, q_gamma, k_gamma, eps, cos_t, sin_t, pos, k_cache, v_cache, nullptr, nullptr,
                                max_seq, use_pdl, stream);
}

// e4m3 cache rows [nkv, max_seq, 128] bytes with scales [nkv, max_seq] fp32
extern "C" int ihb_qk_norm_rope_kv8(float* qkv, int nq, int nkv, const float* q_gamma, const float* k_gamma,
                                    float eps, const float* cos_t, const float* sin_t, const int* pos, void* k_cache,
                                    void* v_cache, float* k_scale, float* v_scale, int max_seq, int use_pdl,
                                    cudaStream_t stream) {
  if (k_scale == nullptr || v_scale == nullptr) return cudaErrorInvalidValue;
  return qk_norm_rope_kv_launch(qkv, nq, nkv, q_gamma, k_gamma, eps, cos_t, sin_t, pos, k_cache, v_cache, k_scale, v_scale,
                                max_seq, use_pdl, stream);
}

extern "C" size_t ihb_flash_decode_scratch_floats(int nq, int nsplit) {
  return static_cast<size_t>(nq) * nsplit * FD_REC;
}

template <bool KV8>
static int flash_decode_launch(const float* q, const void* k_cache, const void* v_cache, const float* k_scale,
                               const float* v_scale, int nq, int nkv, int max_seq, const int* pos, int nsplit,
                               float* scratch, unsigned* counters, float* out, unsigned char* out_q, float* out_s,
                               int out_fp8, int use_pdl, cudaStream_t stream) {
  if (nq % nkv || nsplit < 1 || nsplit > 256) return cudaErrorInvalidValue;
  const int q_per_kv = nq / nkv;
  int gq = q_per_kv >= 8 ? 8 : q_per_kv;
  if (q_per_kv % gq || (gq != 8 && gq != 4 && gq != 2 && gq != 1)) return cudaErrorInvalidValue;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  pdl_cfg(cfg, attr, dim3(nsplit, nkv, q_per_kv / gq), dim3(FD_WARPS * 32), use_pdl, stream);
  switch (gq) {
    case 8: return cudaLaunchKernelEx(&cfg, flash_decode_kernel<8, KV8>, q, k_cache, v_cache, k_scale, v_scale, nq, nkv, max_seq, pos, nsplit, scratch, counters, out, out_q, out_s, out_fp8);
    case 4: return cudaLaunchKernelEx(&cfg, flash_decode_kernel<4, KV8>, q, k_cache, v_cache, k_scale, v_scale, nq, nkv, max_seq, pos, nsplit, scratch, counters, out, out_q, out_s, out_fp8);
    case 2: return cudaLaunchKernelEx(&cfg, flash_decode_kernel<2, KV8>, q, k_cache, v_cache, k_scale, v_scale, nq, nkv, max_seq, pos, nsplit, scratch, counters, out, out_q, out_s, out_fp8);
    default: return cudaLaunchKernelEx(&cfg, flash_decode_kernel<1, KV8>, q, k_cache, v_cache, k_scale, v_scale, nq, nkv, max_seq, pos, nsplit, scratch, counters, out, out_q, out_s, out_fp8);
  }
}

extern "C" int ihb_flash_decode(const float* q, const void* k_cache, const void* v_cache, int nq, int nkv,
                                int max_seq, const int* pos, int nsplit, float* scratch, unsigned* counters,
                                float* out, unsigned char* out_q, float* out_s, int out_fp8, int use_pdl,
                                cudaStream_t stream) {
  return flash_decode_launch<false>(q, k_cache, v_cache, nullptr, nullptr, nq, nkv, max_seq, pos, nsplit, scratch, counters,
                                    out, out_q, out_s, out_fp8, use_pdl, stream);
}

// the same over an e4m3 cache ([nkv, max_seq, 128] bytes, scales [nkv, max_seq] fp32)
extern "C" int ihb_flash_decode_kv8(const float* q, const void* k_cache, const void* v_cache, const float* k_scale,
                                    const float* v_scale, int nq, int nkv, int max_seq, const int* pos, int nsplit,
                                    float* scratch, unsigned* counters, float* out, unsigned char* out_q, float* out_s,
                                    int out_fp8, int use_pdl, cudaStream_t stream) {
  if (k_scale == nullptr || v_scale == nullptr) return cudaErrorInvalidValue;
  return flash_decode_launch<true>(q, k_cache, v_cache, k_scale, v_scale, nq, nkv, max_seq, pos, nsplit, scratch, counters,
                                   out, out_q, out_s, out_fp8, use_pdl, stream);
}

// ---------------------------------------------------------------------------------------------------------------------
// Flash decode for callers that cannot allocate (declared in noalloc.h): the scratch lives in the library image.
// ---------------------------------------------------------------------------------------------------------------------
#include "noalloc.h"
#include <mutex>
#include <stdio.h>

namespace {

constexpr size_t kStaticCounterBytes = 256;   // IHB_FD_STATIC_MAX_HEADS unsigned counters
constexpr size_t kStaticPartialBytes = static_cast<size_t>(IHB_FD_STATIC_MAX_PARTIALS) * ihb::FD_REC * sizeof(float);

// [counters | partials]. In host code this name is only a handle for cudaGetSymbolAddress, never a pointer.
static __device__ __align__(256) unsigned char ihb_fd_static_scratch[kStaticCounterBytes + kStaticPartialBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_static_ptr[kMaxDevices] = {};
std::mutex g_static_mutex;
thread_local char g_static_msg[160] = "";

cudaError_t static_scratch_for_current_device(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, ihb_fd_static_scratch);      // address of this device's copy of the array
    if (e != cudaSuccess) return e;
    g_static_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_static_ptr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" size_t ihb_flash_decode_static_bytes(void) { return kStaticCounterBytes + kStaticPartialBytes; }

extern "C" const char* ihb_flash_decode_static_error(void) { return g_static_msg; }

extern "C" int ihb_flash_decode_static(const float* q, const void* k_cache, const void* v_cache, int nq, int nkv,
                                       int max_seq, const int* pos, int nsplit, float* out, cudaStream_t stream) {
  g_static_msg[0] = '\0';
  if (nq < 1 || nkv < 1 || nsplit < 1 || nq > IHB_FD_STATIC_MAX_HEADS ||
      static_cast<long long>(nq) * nsplit > IHB_FD_STATIC_MAX_PARTIALS) {
    snprintf(g_static_msg, sizeof(g_static_msg),
             "ihb_flash_decode_static: nq=%d, nsplit=%d exceed the built-in scratch (nq <= %d, nq * nsplit <= %d)", nq,
             nsplit, IHB_FD_STATIC_MAX_HEADS, IHB_FD_STATIC_MAX_PARTIALS);
    return cudaErrorInvalidValue;
  }
  // the limits of the kernel itself, checked here so that a refusal comes with a reason and before anything is enqueued
  if (nsplit > IHB_FD_STATIC_MAX_SPLITS) {
    snprintf(g_static_msg, sizeof(g_static_msg), "ihb_flash_decode_static: nsplit=%d exceeds the kernel's limit of %d splits",
             nsplit, IHB_FD_STATIC_MAX_SPLITS);
    return cudaErrorInvalidValue;
  }
  {
    const int per_kv = nq % nkv == 0 ? nq / nkv : 0;
    const bool shape_ok = per_kv > 0 && (per_kv % 8 == 0 || per_kv == 4 || per_kv == 2 || per_kv == 1);
    if (!shape_ok) {
      snprintf(g_static_msg, sizeof(g_static_msg),
               "ihb_flash_decode_static: nq=%d, nkv=%d: query heads per KV head must be 1, 2, 4 or a multiple of 8", nq, nkv);
      return cudaErrorInvalidValue;
    }
  }
  unsigned char* base = nullptr;
  cudaError_t e = static_scratch_for_current_device(&base);
  if (e != cudaSuccess) {
    snprintf(g_static_msg, sizeof(g_static_msg), "ihb_flash_decode_static: no device address for the scratch: %s",
             cudaGetErrorString(e));
    return e;
  }
  // the partials are overwritten before they are read; only the arrival counters have to start at zero
  e = cudaMemsetAsync(base, 0, kStaticCounterBytes, stream);
  if (e != cudaSuccess) {
    snprintf(g_static_msg, sizeof(g_static_msg), "ihb_flash_decode_static: clearing the arrival counters failed: %s",
             cudaGetErrorString(e));
    return e;
  }
  const int rc = ihb_flash_decode(q, k_cache, v_cache, nq, nkv, max_seq, pos, nsplit,
                                  reinterpret_cast<float*>(base + kStaticCounterBytes), reinterpret_cast<unsigned*>(base), out,
                                  nullptr, nullptr, 0, 0, stream);
  if (rc != cudaSuccess)
    snprintf(g_static_msg, sizeof(g_static_msg), "ihb_flash_decode_static: the launch failed: %s",
             cudaGetErrorString(static_cast<cudaError_t>(rc)));
  return rc;
}
