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
  // optional copy of the normed vector as the tensor-core kernels' activation operand: plain row of e4m3
  // bytes with one fp32 scale per 128 channels (xq_fp8 = 1), or a bf16 row (xq_fp8 = 0); nullptr = none
  uint8_t* xq;
  float* xs;
  int xq_fp8;
};

// Quantise 4 consecutive values per lane (a warp = one group of 128 channels) to e4m3 with scale amax / 448.
__device__ __forceinline__ void quant_group128(float4 v, uint8_t* dst4, float* scale_out, int lane) {
  float m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
  m = warp_max(m);
  const float s = fmaxf(m, 1e-12f) * (1.f / 448.f);
  const float inv = 1.f / s;
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v.x * inv, v.y * inv), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v.z * inv, v.w * inv), __NV_SATFINITE, __NV_E4M3);
  *reinterpret_cast<uint32_t*>(dst4) = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
  if (lane == 0) *scale_out = s;
}
__device__ __forceinline__ void store_bf16x4(float4 v, uint8_t* dst8) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 o;
  o.x = *reinterpret_cast<const uint32_t*>(&a);
  o.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(dst8) = o;
}

// Runs in the consumer threads of the last CTA: cross-GPU arrive/wait, sum of all slots in slot order,
// residual add, RMSNorm. Every rank sums the same values in the same order, so the replicated residual stream
// stays bitwise identical across ranks.
template <int NTHR, int BAR>
__device__ __forceinline__ void tail_ar_norm(const ArNormTail& a, int tid, float* red_smem) {
  const IhbComm& cm = a.comm;
  const int H = a.H;
  const unsigned epoch = *cm.epoch;
  const int parity = epoch & 1u;
  if (cm.nranks > 1) {
    if (tid == 0) peer_barrier(cm, (epoch + 1u) * static_cast<unsigned>(cm.nranks), a.err);
    named_bar_sync(BAR, NTHR);
  }
  const int nslots = cm.nranks * a.ks;
  const float* slots = cm.slots_local + static_cast<size_t>(parity) * nslots * H;
  constexpr int MAXV = 8192 / 4 / NTHR;          // H <= 8192: float4s per thread, kept in registers
  float4 acc[MAXV];
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = (tid + NTHR * j) * 4;
    acc[j] = (i < H) ? *reinterpret_cast<const float4*>(a.resid + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int s = 0; s < nslots; ++s) {
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int i = (tid + NTHR * j) * 4;
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
  named_bar_sync(BAR, NTHR);
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < NTHR / 32; ++w) tot += red_smem[w];
  const float rinv = rsqrtf(tot / static_cast<float>(H) + a.eps);
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = (tid + NTHR * j) * 4;
    if (i < H) {
      const float4 g = *reinterpret_cast<const float4*>(a.gamma + i);
      *reinterpret_cast<float4*>(a.resid + i) = acc[j];
      const float4 o = make_float4(acc[j].x * rinv * g.x, acc[j].y * rinv * g.y, acc[j].z * rinv * g.z,
                                   acc[j].w * rinv * g.w);
      *reinterpret_cast<float4*>(a.xn_out + i) = o;
      if (a.xq != nullptr) {          // H is a multiple of 128, so a warp is entirely inside or outside
        if (a.xq_fp8) quant_group128(o, a.xq + i, a.xs + (i >> 7), tid & 31);
        else store_bf16x4(o, a.xq + 2 * i);
      }
    }
  }
  if (tid == 0) *cm.epoch = epoch + 1u;
}


struct ArgmaxTail {
  IhbComm comm;
  unsigned long long* argmax_partial;   // one packed (value, local row) per CTA
  int nblocks;
  int vocab0;
  int* cur_token;
  int* pos;
  int* token_ring;
  int token_ring_size;
  const int* forced;
  const int* n_forced;
  unsigned* err;
};

// Last CTA: global argmax over the per-CTA maxima (and over the ranks of a vocabulary-sharded head), next token
// and position counter update.
template <int NTHR, int BAR>
__device__ __forceinline__ void tail_argmax(const ArgmaxTail& a, int tid, unsigned long long* red_smem) {
  const int nblocks = a.nblocks;
  unsigned long long best = 0ull;
  for (int i = tid; i < nblocks; i += NTHR) {
    const unsigned long long p = ld_cg_u64(a.argmax_partial + i);
    best = p > best ? p : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long q = __shfl_xor_sync(0xffffffffu, best, o);
    best = q > best ? q : best;
  }
  if ((tid & 31) == 0) red_smem[tid >> 5] = best;
  named_bar_sync(BAR, NTHR);
  if (tid == 0) {
#pragma unroll
    for (int w = 0; w < NTHR / 32; ++w) best = red_smem[w] > best ? red_smem[w] : best;
    const IhbComm& cm = a.comm;
    // local winner carries the GLOBAL token id so that ties across ranks resolve to the lowest id
    unsigned long long mine = (best & 0xffffffff00000000ull) |
                              (0xffffffffu - (unpack_idx(best) + static_cast<unsigned>(a.vocab0)));
    if (cm.nranks > 1) {
      const unsigned epoch = *cm.epoch;
      const int parity = epoch & 1u;
      unsigned long long* slot_local = cm.arg_slots_local + parity * cm.nranks;
      if (cm.arg_slots_mc != nullptr) {
        multimem_st_u64(cm.arg_slots_mc + parity * cm.nranks + cm.rank, mine);
      } else {
        for (int r = 0; r < cm.nranks; ++r)
          st_relaxed_sys_u64(cm.arg_slots_peer[r] + parity * cm.nranks + cm.rank, mine);
      }
      peer_barrier(cm, (epoch + 1u) * static_cast<unsigned>(cm.nranks), a.err);
      for (int r = 0; r < cm.nranks; ++r) {
        const unsigned long long p = ld_cg_u64(slot_local + r);
        mine = p > mine ? p : mine;
      }
      *cm.epoch = epoch + 1u;
    }
    const int tok = static_cast<int>(unpack_idx(mine));
    const int pos = *a.pos;
    int next = tok;
    if (a.forced != nullptr && pos + 1 < *a.n_forced) next = a.forced[pos + 1];
    *a.cur_token = next;
    if (a.token_ring != nullptr) a.token_ring[pos % a.token_ring_size] = tok;
    *a.pos = pos + 1;
  }
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
