// All-to-all exchange of rows over peer memory: the dispatch / combine primitive of expert parallelism for windows of
// several tokens (prompt chunks, verify windows), where each rank routes only its own tokens.
//
// ONE kernel per exchange. Every rank holds P rows sorted by destination (or a gather list into an unsorted matrix:
// the permutation is fused into the send). CTAs copy row p straight into the destination GPU's receive region
// [parity][source rank][slot][row] with 16-byte peer stores, CTA 0 stores the per-destination counts beside it, then
// every CTA fences, adds itself to every GPU's arrival counter and waits (bounded) until all ranks x CTAs of this
// round have arrived on its own counter: after the kernel the local receive region and counts are complete. Two
// parities are enough because a rank starts round n + 1 only after the work that consumed round n on its stream.
// The launch is cooperative: the CTAs wait for other GPUs, so all of them must be resident.
//
// The reference has this primitive only on NVSHMEM (kernels/nvshmem_comms.cu:170-191: PE i puts chunk j into PE j's
// recv[i * CHUNK], one barrier) and combines expert outputs with an NCCL all-reduce (kernels/ep_moe_sharded.cu:309-337).
#include "common.cuh"
#include "api.h"

namespace ihb {

constexpr int A2A_THREADS = 256;

__global__ void __launch_bounds__(A2A_THREADS) a2a_rows_kernel(const IhbA2AArgs a) {
  const int nr = a.nranks;
  const unsigned parity = a.round & 1u;
  const int rf4 = a.row_floats / 4;
  __shared__ int off_s[IHB_MAX_RANKS + 1];
  if (threadIdx.x <= nr) off_s[threadIdx.x] = a.offsets[threadIdx.x];
  __syncthreads();
  const int P = off_s[nr];
  // rows: CTA-strided over pairs, threads over the 16-byte pieces of a row
  for (int p = blockIdx.x; p < P; p += gridDim.x) {
    int d = 0;
    while (d + 1 < nr && p >= off_s[d + 1]) ++d;
    const int slot = p - off_s[d];
    if (slot >= a.cap) {                          // the caller sized the slots too small: report, skip the row
      if (threadIdx.x == 0) set_error(a.err, ERR_BAD_ARGS);
      continue;
    }
    const int src_row = a.gather != nullptr ? a.gather[p] : p;
    const float4* src = reinterpret_cast<const float4*>(a.send + static_cast<size_t>(src_row) * a.row_floats);
    float4* dst = reinterpret_cast<float4*>(a.recv_peer[d] +
                                            ((static_cast<size_t>(parity) * nr + a.rank) * a.cap + slot) * a.row_floats);
    for (int i = threadIdx.x; i < rf4; i += A2A_THREADS) dst[i] = src[i];
  }
  if (blockIdx.x == 0 && threadIdx.x < nr) {
    const int d = threadIdx.x;
    a.count_peer[d][parity * nr + a.rank] = min(off_s[d + 1] - off_s[d], a.cap);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // the CTA's stores (ordered before this thread by the barrier) become visible to whoever acquires the counter
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    for (int r = 0; r < nr; ++r) red_release_sys_add_u32(a.flag_peer[r], 1u);
    wait_flag_ge(a.flag_local, (a.round + 1u) * static_cast<unsigned>(nr) * gridDim.x, a.err, ERR_PEER_BARRIER_TIMEOUT);
  }
  __syncthreads();
}

}  // namespace ihb

using namespace ihb;

extern "C" int ihb_a2a_rows(const IhbA2AArgs* args, int grid, cudaStream_t stream) {
  if (args == nullptr || args->nranks < 1 || args->nranks > IHB_MAX_RANKS || args->row_floats < 4 ||
      (args->row_floats % 4) || args->cap < 1 || args->offsets == nullptr)      // send may be NULL when no row is sent
    return cudaErrorInvalidValue;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (grid <= 0) grid = 32;
  if (grid > sms) grid = sms;                      // the CTAs wait on other GPUs: all must be resident
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(A2A_THREADS);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, a2a_rows_kernel, *args);
}
