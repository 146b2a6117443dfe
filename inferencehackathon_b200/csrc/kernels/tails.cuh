// Epilogue "tails" run by the last CTA of a streaming kernel: cross-GPU barrier, slot reduction + residual +
// RMSNorm, packed (value, index) maxima.
#pragma once
#include "common.cuh"
#include "api.h"

namespace ihb {

__device__ __forceinline__ unsigned long long pack_max(float v, unsigned idx) {
  unsigned b = __float_as_uint(v);
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);   // monotonic map float -> unsigned
  return (static_cast<unsigned long long>(b) << 32) | (0xffffffffu - idx);
}
__device__ __forceinline__ unsigned unpack_idx(unsigned long long p) { return 0xffffffffu - static_cast<unsigned>(p); }

// ---- tails -------------------------------------------------------------------------------------------------------

// Cross-GPU arrive + wait on a monotonic counter (one thread). Returns false on time-out.
__device__ __forceinline__ bool peer_barrier(const IhbComm& cm, unsigned target, unsigned* err) {
  __threadfence_system();
  if (cm.flag_mc != nullptr) {
    multimem_red_release_sys_add_u32(cm.flag_mc, 1u);
  } else {
    for (int r = 0; r < cm.nranks; ++r) red_release_sys_add_u32(cm.flag_peer[r], 1u);
  }
  return wait_flag_ge(cm.flag_local, target, err, ERR_PEER_BARRIER_TIMEOUT);
}

struct ArNormTail {
  IhbComm comm;
  int H;
  int ks;            // partial slots per rank (K-split factor of the producing kernel)
  float* resid;
  const float* gamma;
  float* xn_out;
  float eps;
  unsigned* err;
};

// Runs in the consumer threads of the last CTA: cross-GPU arrive/wait, sum of all slots in slot order,
// residual add, RMSNorm. Every rank sums the same values in the same order, so the replicated residual stream
// stays bitwise identical across ranks.
__device__ __forceinline__ void tail_ar_norm(const ArNormTail& a, int tid, float* red_smem) {
  const IhbComm& cm = a.comm;
  const int H = a.H;
  const unsigned epoch = *cm.epoch;
  const int parity = epoch & 1u;
  if (cm.nranks > 1) {
    if (tid == 0) peer_barrier(cm, (epoch + 1u) * static_cast<unsigned>(cm.nranks), a.err);
    named_bar_sync(1, CONSUMER_THREADS);
  }
  const int nslots = cm.nranks * a.ks;
  const float* slots = cm.slots_local + static_cast<size_t>(parity) * nslots * H;
  constexpr int MAXV = 8;                       // H <= 8192: at most 8 float4 per thread, kept in registers
  float4 acc[MAXV];
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = (tid + CONSUMER_THREADS * j) * 4;
    acc[j] = (i < H) ? *reinterpret_cast<const float4*>(a.resid + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int s = 0; s < nslots; ++s) {
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int i = (tid + CONSUMER_THREADS * j) * 4;
      if (i < H) {
        const float4 v = ld_cg_f4(reinterpret_cast<const float4*>(slots + static_cast<size_t>(s) * H + i));
        acc[j].x += v.x; acc[j].y += v.y; acc[j].z += v.z; acc[j].w += v.w;
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAXV; ++j)
    ss += acc[j].x * acc[j].x + acc[j].y * acc[j].y + acc[j].z * acc[j].z + acc[j].w * acc[j].w;
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red_smem[tid >> 5] = ss;
  named_bar_sync(1, CONSUMER_THREADS);
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < NCW; ++w) tot += red_smem[w];
  const float rinv = rsqrtf(tot / static_cast<float>(H) + a.eps);
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = (tid + CONSUMER_THREADS * j) * 4;
    if (i < H) {
      const float4 g = *reinterpret_cast<const float4*>(a.gamma + i);
      *reinterpret_cast<float4*>(a.resid + i) = acc[j];
      *reinterpret_cast<float4*>(a.xn_out + i) =
          make_float4(acc[j].x * rinv * g.x, acc[j].y * rinv * g.y, acc[j].z * rinv * g.z, acc[j].w * rinv * g.w);
    }
  }
  if (tid == 0) *cm.epoch = epoch + 1u;
}


// Push one partial output value into slot `slot` of every GPU's buffer (or the local one).
__device__ __forceinline__ void push_partial(const IhbComm& cm, size_t off, float y) {
  if (cm.nranks == 1) {
    cm.slots_local[off] = y;
  } else if (cm.slots_mc != nullptr) {
    multimem_st_f32(cm.slots_mc + off, y);
  } else {
    for (int p = 0; p < cm.nranks; ++p) st_relaxed_sys_f32(cm.slots_peer[p] + off, y);
  }
}

}  // namespace ihb
