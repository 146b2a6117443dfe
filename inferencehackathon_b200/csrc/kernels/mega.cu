// Persistent decode megakernel: ONE cooperative launch runs whole tokens - every layer's QKV GEMV, QK-norm + RoPE +
// KV append + split-KV attention, o_proj, router + top-k, expert gate/up + SwiGLU, expert down, the two
// tensor-parallel all-reduces (partials added straight into every GPU's slot buffer through NVSwitch, multimem.red or
// peer reds) with residual + RMSNorm, the final norm, the vocabulary-sharded head and the cross-rank argmax.
//
// Why: at one token a tensor-parallel layer moves only a few MB per GPU, so a chain of separate kernels is bound
// by launch, prologue and tail latencies, not by bytes. Here a phase hands its result to the next one as tagged
// values the consumer waits on; the two all-reduces of a layer are counted fixed-point accumulations (every rank adds
// its partial into every GPU's slot with one multimem.red / peer red, the reader waits for the contribution count);
// the residual stream lives in every CTA's shared memory (all CTAs read the same integer sums, so the copies stay
// bitwise identical on every CTA of every GPU) and the activation vector of each GEMV is staged once per CTA in
// shared memory as pre-scaled fp16.
//
// All CTAs must be resident (cooperative launch, one per SM). Every wait is bounded: on a time-out the error word is
// set, all later waits fall through and the kernel ends normally.
//
// The reference's persistent kernel (kernels/megakernel_decode.cu:575-649) pays ~16 cooperative grid syncs and
// NVSHMEM barriers per layer and measured 9-11x slower than its multi-kernel path (docs/path-to-1000.md:32-34).
#include <algorithm>
#include "common.cuh"
#include "tails.cuh"

// The body is compiled twice, into ihb::narrow and ihb::wide. In both, the warps that produce a gate / up row pair apply
// SwiGLU and the routing weight themselves (MG_PAIR: the down phase then reads half as many hand-over values; -1.6 % per
// token at TP8 shapes, -2 % at TP4). The wide build adds a GEMV shape for CTAs that own many rows per warp: with it a
// full-width model on one GPU runs 9 % faster and TP2 2 %, but compiled into the same kernel that code costs the
// shapes of TP4 / TP8 3-7 % (instruction-cache footprint and register pressure in every function that inlines the
// shape helpers), so the host picks the build by the size of the expert GEMV's shares (mega_host.inc::mega_wide).
#ifndef MG_NARROW_PAIR
#define MG_NARROW_PAIR 1
#endif
#define MG_NS narrow
#define MG_WIDE 0
#define MG_PAIR MG_NARROW_PAIR
#include "mega_body.inc"
#undef MG_NS
#undef MG_WIDE
#undef MG_PAIR
#define MG_NS wide
#define MG_WIDE 1
#define MG_PAIR 1
#include "mega_body.inc"
#undef MG_NS
#undef MG_WIDE
#undef MG_PAIR

#include "mega_host.inc"
