// Weight-streaming pipeline shared by the decode GEMV kernels.
//
// One producer warp feeds a ring of shared-memory stages with bulk asynchronous copies (the TMA engine moves
// whole row tiles, `cp.async.bulk`, completion counted on an mbarrier); eight consumer warps take one weight
// row per warp with the activation vector held in registers. At batch 1 the kernel is a pure HBM stream, so
// the design goal is to keep ~100-190 KB of copies in flight per SM and to spend the fewest issue slots per
// byte: hardware e4m3x2->f16x2 conversion and packed HFMA2, one fp32 scale multiply per 16 weights.
//
// The reference's GEMV idiom is a warp per row with direct `uint4` global loads and fp32 FMAs
// (kernels/k5_experts.cu:55-82), measured at 45-58 % of H100 bandwidth (docs/k5-kernel-results-h100.md:21-32).
#pragma once
#include "common.cuh"

namespace ihb {

struct Ring {
  uint64_t* full;    // [S]
  uint64_t* empty;   // [S]
  uint8_t* stages;   // S * stage_stride bytes
  int S;
  int stage_stride;
};

// Carves the dynamic shared memory: [full S][empty S] | pad to 256 | stages. Returns the ring; thread 0
// initialises the barriers (`empty_count` consumer arrivals free a stage).
__device__ __forceinline__ Ring ring_setup(uint8_t* smem, int S, int stage_stride, int tid, int empty_count) {
  Ring r;
  r.full = reinterpret_cast<uint64_t*>(smem);
  r.empty = r.full + S;
  r.stages = smem + 256;   // 2 S barriers of 8 bytes fit in the first 256 bytes (S <= 12)
  r.S = S;
  r.stage_stride = stage_stride;
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&r.full[s], 1);
      mbar_init(&r.empty[s], empty_count);
    }
    fence_mbar_init();
  }
  return r;
}

// Activation fragment of one lane: a row is shared by G adjacent lanes (G = 32: a warp per row), lane g of the
// group takes chunks c = g + G i, chunk c covering elements [16 c, 16 c + 16) (fp8 weights) of the K-slice at `x`.
template <int NI>
struct XFragF16 {
  uint4 lo[NI], hi[NI];
  float unscale;   // multiply results by this to undo the power-of-two pre-scale

  __device__ __forceinline__ void load(const float* __restrict__ x, int nchunks, int g, int G = 32) {
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int c = g + G * i;
      if (c < nchunks) {
        const float4* p = reinterpret_cast<const float4*>(x + 16 * c);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 v = ld_cg_f4(p + j);
          m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
      }
    }
    m = warp_max(m);
    // power-of-two scale that brings max|x| to at most 8
    int e = 0;
    if (m > 8.f) e = static_cast<int>(ceilf(log2f(m * 0.125f)));
    const float s = exp2f(static_cast<float>(-e));
    unscale = exp2f(static_cast<float>(e));
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int c = g + G * i;
      lo[i] = make_uint4(0, 0, 0, 0);
      hi[i] = make_uint4(0, 0, 0, 0);
      if (c < nchunks) {
        const float4* p = reinterpret_cast<const float4*>(x + 16 * c);
        const float4 a = ld_cg_f4(p), b = ld_cg_f4(p + 1), cc = ld_cg_f4(p + 2), d = ld_cg_f4(p + 3);
        __half2 h;
        h = __floats2half2_rn(a.x * s, a.y * s);  lo[i].x = *reinterpret_cast<unsigned*>(&h);
        h = __floats2half2_rn(a.z * s, a.w * s);  lo[i].y = *reinterpret_cast<unsigned*>(&h);
        h = __floats2half2_rn(b.x * s, b.y * s);  lo[i].z = *reinterpret_cast<unsigned*>(&h);
        h = __floats2half2_rn(b.z * s, b.w * s);  lo[i].w = *reinterpret_cast<unsigned*>(&h);
        h = __floats2half2_rn(cc.x * s, cc.y * s); hi[i].x = *reinterpret_cast<unsigned*>(&h);
        h = __floats2half2_rn(cc.z * s, cc.w * s); hi[i].y = *reinterpret_cast<unsigned*>(&h);
        h = __floats2half2_rn(d.x * s, d.y * s);  hi[i].z = *reinterpret_cast<unsigned*>(&h);
        h = __floats2half2_rn(d.z * s, d.w * s);  hi[i].w = *reinterpret_cast<unsigned*>(&h);
      }
    }
  }
};

// Same for bf16 weights: chunk c covers elements [8 c, 8 c + 8), activations stay fp32.
template <int NI>
struct XFragF32 {
  float4 a[NI], b[NI];
  float unscale;

  __device__ __forceinline__ void load(const float* __restrict__ x, int nchunks, int g, int G = 32) {
    unscale = 1.f;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int c = g + G * i;
      a[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      b[i] = a[i];
      if (c < nchunks) {
        const float4* p = reinterpret_cast<const float4*>(x + 8 * c);
        a[i] = ld_cg_f4(p);
        b[i] = ld_cg_f4(p + 1);
      }
    }
  }
};

// Dot product of one (virtual) weight row in shared memory with the register fragment.
// `row` points at the row's first byte for this K-slice; `sc` at the row block's scales for this slice
// (fp8 only), `kb_shift` = log2 of the scale block width in 16-element chunks.
template <int NI>
__device__ __forceinline__ float row_dot_fp8(const uint8_t* row, const XFragF16<NI>& xf, const float* sc,
                                             int chunk0, int kb_shift, int nchunks, int lane) {
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int c = lane + 32 * i;
    if (c < nchunks) {
      const uint4 w = *reinterpret_cast<const uint4*>(row + 16 * c);
      const float s = sc[(chunk0 + c) >> kb_shift];
      acc = fmaf(s, dot16_e4m3(w, xf.lo[i], xf.hi[i]), acc);
    }
  }
  return warp_sum(acc) * xf.unscale;
}

template <int NI>
__device__ __forceinline__ float row_dot_bf16(const uint8_t* row, const XFragF32<NI>& xf, int nchunks, int lane) {
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int c = lane + 32 * i;
    if (c < nchunks) {
      const uint4 w = *reinterpret_cast<const uint4*>(row + 16 * c);
      acc += dot8_bf16(w, xf.a[i], xf.b[i]);
    }
  }
  return warp_sum(acc);
}

// Variants for rows shared by G < 32 lanes (short rows): lanes [q G, q G + G) of a warp work on one row; the sum
// runs over the group only.
__device__ __forceinline__ float group_sum(float v, int G) {
  for (int o = G >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int NI>
__device__ __forceinline__ float group_dot_fp8(const uint8_t* row, const XFragF16<NI>& xf, const float* sc,
                                               int kb_shift, int nchunks, int g, int G) {
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int c = g + G * i;
    if (c < nchunks) {
      const uint4 w = *reinterpret_cast<const uint4*>(row + 16 * c);
      acc = fmaf(sc[c >> kb_shift], dot16_e4m3(w, xf.lo[i], xf.hi[i]), acc);
    }
  }
  return group_sum(acc, G) * xf.unscale;
}

template <int NI>
__device__ __forceinline__ float group_dot_bf16(const uint8_t* row, const XFragF32<NI>& xf, int nchunks, int g, int G) {
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int c = g + G * i;
    if (c < nchunks) {
      const uint4 w = *reinterpret_cast<const uint4*>(row + 16 * c);
      acc += dot8_bf16(w, xf.a[i], xf.b[i]);
    }
  }
  return group_sum(acc, G);
}

}  // namespace ihb
