// Shared device helpers for the sm_100a decode kernels: mbarrier pipeline primitives with bounded waits, bulk
// asynchronous (TMA engine) global->shared copies, programmatic dependent launch control, system-scope
// release/acquire and NVLS multimem accesses, fp8/bf16 dot-product fragments.
//
// Every wait in this file gives up after a time limit, records a code in a device error word and lets the
// kernel run to its normal end (the reference's spins are unbounded, kernels/nvls_engine.cuh:137-139,
// kernels/oneshot_allreduce.cu:151-153).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace ihb {

// ---- error reporting ------------------------------------------------------------------------------------------
enum ErrCode : unsigned {
  ERR_NONE = 0,
  ERR_MBAR_FULL_TIMEOUT = 1,
  ERR_MBAR_EMPTY_TIMEOUT = 2,
  ERR_PEER_BARRIER_TIMEOUT = 3,
  ERR_GRID_COUNTER_TIMEOUT = 4,
  ERR_TMEM_TIMEOUT = 5,
  ERR_BAD_ARGS = 6,
};

// Wait limits in nanoseconds of %globaltimer. Intra-SM pipeline waits are short; waits on another GPU get a
// second (a rank that stopped answering must not hold this GPU).
#ifndef IHB_LOCAL_WAIT_NS
#define IHB_LOCAL_WAIT_NS 2000000000ull
#endif
#ifndef IHB_PEER_WAIT_NS
#define IHB_PEER_WAIT_NS 1000000000ull
#endif

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void set_error(unsigned* err, unsigned code) {
  if (err != nullptr) atomicCAS(err, 0u, code);
}

// ---- shared memory / mbarrier ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait on a phase of an mbarrier. Returns false (and records `code`) when the limit passes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned* err, unsigned code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 255u) == 0u && globaltimer_ns() - t0 > IHB_LOCAL_WAIT_NS) {
      set_error(err, code);
      return false;
    }
  }
  return true;
}

// Bulk asynchronous copy global -> shared, completion counted in bytes on `bar`. `dst`, `src` 16-byte aligned,
// `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// ---- programmatic dependent launch -------------------------------------------------------------------------------
// wait: all memory of the kernels this launch depends on is visible afterwards (no-op without the attribute).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Allow the next kernel in the stream to begin its prologue. Issued only after pdl_wait() so that "the
// previous kernel has completed" holds transitively for every later kernel's prologue.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- named barriers (consumer warps only; the producer warp never joins) -----------------------------------------
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- global memory accesses that bypass L1 (data written by other SMs / other GPUs) --------------------------------
__device__ __forceinline__ float4 ld_cg_f4(const float4* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_cg_f(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ int ld_cg_i(const int* p) {
  int v;
  asm volatile("ld.global.cg.s32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ unsigned ld_cg_u(const unsigned* p) {
  unsigned v;
  asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ unsigned long long ld_cg_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.global.cg.u64 %0, [%1];" : "=l"(v) : "l"(p));
  return v;
}

// ---- system scope signalling between GPUs ----------------------------------------------------------------------
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add_u32(unsigned* p, unsigned v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// NVLS: one instruction, the switch applies it to every GPU bound to the multicast address.
__device__ __forceinline__ void multimem_red_release_sys_add_u32(unsigned* mc, unsigned v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_st_f32(float* mc, float v) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc), "f"(v) : "memory");
}
__device__ __forceinline__ void multimem_st_f4(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ void multimem_st_u64(unsigned long long* mc, unsigned long long v) {
  asm volatile("multimem.st.relaxed.sys.global.b64 [%0], %1;" ::"l"(mc), "l"(v) : "memory");
}
__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_f32(float* p, float v) {
  asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Bounded spin until *flag (monotonic counter, compared on the signed difference so that wrap-around is safe)
// reaches `target`. Returns false on time-out.
__device__ __forceinline__ bool wait_flag_ge(const unsigned* flag, unsigned target, unsigned* err, unsigned code) {
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (static_cast<int>(ld_acquire_sys_u32(flag) - target) < 0) {
    if ((++spins & 63u) == 0u && globaltimer_ns() - t0 > IHB_PEER_WAIT_NS) {
      set_error(err, code);
      return false;
    }
  }
  return true;
}

// ---- math fragments -------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ __half2 cvt_e4m3x2(unsigned short v) {
  __half2_raw r = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(v), __NV_E4M3);
  return *reinterpret_cast<__half2*>(&r);
}

// four e4m3 bytes of one 32-bit word (lowest byte first) as floats
__device__ __forceinline__ float4 e4m3x4_to_float4(unsigned w) {
  const float2 a = __half22float2(cvt_e4m3x2(static_cast<unsigned short>(w & 0xffffu)));
  const float2 b = __half22float2(cvt_e4m3x2(static_cast<unsigned short>(w >> 16)));
  return make_float4(a.x, a.y, b.x, b.y);
}

// One warp stores a KV-cache row of 128 channels (lane holds channels lane + 32 j). KV8: e4m3 bytes plus one fp32 scale
// per row (amax / 448, the per-(head, position) scheme of the PyTorch cache of this package); otherwise bf16.
template <bool KV8>
__device__ __forceinline__ void kv_store_row(void* cache, float* scale, size_t row, const float (&x)[4], int lane) {
  if constexpr (KV8) {
    const float amax = warp_max(fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3]))));
    const float sc = fmaxf(amax, 1e-12f) / 448.f;
    uint8_t* dst = reinterpret_cast<uint8_t*>(cache) + row * 128;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      dst[lane + 32 * j] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(x[j] / sc, __NV_SATFINITE, __NV_E4M3));
    if (lane == 0) scale[row] = sc;
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(cache) + row * 128;
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[lane + 32 * j] = __float2bfloat16(x[j]);
  }
}

// 16 e4m3 weights (one uint4) times 16 fp16 activations (two uint4: elements 0-7 and 8-15), fp32 result.
// Products accumulate in two fp16x2 chains of four; activations are pre-scaled by the caller so that
// |x| <= 8, which bounds each chain by 4 * 448 * 8 < 65504.
__device__ __forceinline__ float dot16_e4m3(uint4 w, uint4 xlo, uint4 xhi) {
  const __half2* xl = reinterpret_cast<const __half2*>(&xlo);
  const __half2* xh = reinterpret_cast<const __half2*>(&xhi);
  __half2 a = __float2half2_rn(0.f), b = __float2half2_rn(0.f);
  a = __hfma2(cvt_e4m3x2(w.x & 0xffffu), xl[0], a);
  b = __hfma2(cvt_e4m3x2(w.x >> 16), xl[1], b);
  a = __hfma2(cvt_e4m3x2(w.y & 0xffffu), xl[2], a);
  b = __hfma2(cvt_e4m3x2(w.y >> 16), xl[3], b);
  a = __hfma2(cvt_e4m3x2(w.z & 0xffffu), xh[0], a);
  b = __hfma2(cvt_e4m3x2(w.z >> 16), xh[1], b);
  a = __hfma2(cvt_e4m3x2(w.w & 0xffffu), xh[2], a);
  b = __hfma2(cvt_e4m3x2(w.w >> 16), xh[3], b);
  const float2 fa = __half22float2(a), fb = __half22float2(b);
  return (fa.x + fa.y) + (fb.x + fb.y);
}

// 8 bf16 weights (one uint4) times 8 fp32 activations.
__device__ __forceinline__ float dot8_bf16(uint4 w, float4 x0, float4 x1) {
  float acc;
  acc = __uint_as_float(w.x << 16) * x0.x;
  acc = fmaf(__uint_as_float(w.x & 0xffff0000u), x0.y, acc);
  acc = fmaf(__uint_as_float(w.y << 16), x0.z, acc);
  acc = fmaf(__uint_as_float(w.y & 0xffff0000u), x0.w, acc);
  acc = fmaf(__uint_as_float(w.z << 16), x1.x, acc);
  acc = fmaf(__uint_as_float(w.z & 0xffff0000u), x1.y, acc);
  acc = fmaf(__uint_as_float(w.w << 16), x1.z, acc);
  acc = fmaf(__uint_as_float(w.w & 0xffff0000u), x1.w, acc);
  return acc;
}

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

// Launch geometry shared by the streaming kernels: one producer warp + NCW consumer warps.
constexpr int NCW = 8;
constexpr int CONSUMER_THREADS = NCW * 32;
constexpr int STREAM_THREADS = CONSUMER_THREADS + 32;

}  // namespace ihb
