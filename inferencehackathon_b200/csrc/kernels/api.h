// C ABI of the sm_100a kernel library (loaded from Python with ctypes; every entry launches on the given
// stream and returns a cudaError_t value, 0 = success). All pointers are device pointers unless noted.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IHB_MAX_RANKS 8
#define IHB_MAX_TOPK 8

enum { IHB_W_FP8 = 0, IHB_W_BF16 = 1 };
enum { IHB_EPI_STORE = 0, IHB_EPI_ROUTER = 1, IHB_EPI_ARGMAX = 2, IHB_EPI_AR_NORM = 3 };

// Cross-GPU state of the fused all-reduce epilogues. With nranks == 1 only slots_local and epoch are used.
// Multicast mode: *_mc are NVLS multicast addresses of the same symmetric buffers (one store reaches every
// GPU); peer mode (*_mc == NULL): *_peer[r] is rank r's buffer mapped into this process.
typedef struct {
  int nranks;
  int rank;
  float* slots_local;                        // [2][nranks * ks][H] fp32 partials, double buffered by epoch parity
                                             // (persistent kernel: [8 round parities][H] 64-bit counted fixed-point
                                             // sums, zero-initialised)
  float* slots_mc;
  float* slots_peer[IHB_MAX_RANKS];
  unsigned* flag_local;                      // monotonic arrival counter
  unsigned* flag_mc;
  unsigned* flag_peer[IHB_MAX_RANKS];
  unsigned long long* arg_slots_local;       // [2][nranks] packed (value, token) for the sharded head
  unsigned long long* arg_slots_mc;
  unsigned long long* arg_slots_peer[IHB_MAX_RANKS];
  unsigned* epoch;                           // local, 4 words: [0] collectives completed so far, [1] rounds of the
                                             // arrival counter made by the persistent kernel
} IhbComm;

typedef struct {
  // weights
  const uint8_t* W;        // [rows, K] e4m3 bytes or bf16, rows contiguous
  const float* wscale;     // fp8: [ceil(rows / rb), nkb]
  int wtype;               // IHB_W_*
  int rows, K;
  int rb, kb_shift, nkb;   // scale block: rb rows x (1 << kb_shift) columns
  // input
  const float* x;          // [K] fp32
  // tiling (0 = choose)
  int R, S, grid, ks;      // rows per tile, ring stages, CTAs, K-split (AR_NORM only)
  int epi;                 // IHB_EPI_*
  float* out;              // STORE / ROUTER / (ARGMAX, optional): [rows] fp32
  unsigned* counter;       // last-CTA election word (zero before the first launch)
  unsigned* err;           // device error word (0 = none)
  // ROUTER
  int top_k, renorm;
  int* sel_idx;            // [top_k]
  float* sel_w;            // [top_k]
  float* router_partial;   // ROUTER with ks > 1: [ks][rows] partial logits, summed in order by the tail
  // ARGMAX
  unsigned long long* argmax_partial;   // [grid]
  int vocab0;
  int* cur_token;          // next input token
  int* pos;                // position counter, incremented by the tail
  int* token_ring;         // optional ring of generated tokens indexed by position
  int token_ring_size;
  const int* forced;       // optional: tokens that override the argmax while position + 1 < *n_forced (prompt replay)
  const int* n_forced;
  // AR_NORM
  float* resid;            // [rows] residual stream, updated in place
  const float* gamma;      // [rows] weight of the norm that follows
  float* xn_out;           // [rows] normed output
  float eps;
  IhbComm comm;
} IhbGemvArgs;

int ihb_gemv(IhbGemvArgs* args, int use_pdl, cudaStream_t stream);

// MoE expert kernels (M = 1). Expert ids / weights come from device memory (the router tail wrote them).
typedef struct {
  const uint8_t* Wgu;      // [E_local, 2 * I, H]: gate rows then up rows
  const float* gu_scale;   // fp8: [E_local, ceil(2 I / rb), nkb]
  const uint8_t* Wd;       // [E_local, H, I]
  const float* d_scale;    // fp8: [E_local, ceil(H / d_rb), d_nkb]
  int wtype;
  int H, I, E_local, expert0, top_k;
  int gu_rb, gu_kb_shift, gu_nkb;
  int d_rb, d_kb_shift, d_nkb;
  const float* x;          // [H] normed hidden
  const int* sel_idx;      // [top_k] global expert ids
  const float* sel_w;      // [top_k]
  float* act;              // [top_k, I] fp32 SwiGLU activations (scratch between the two kernels)
  int R_gu, R_d, S, grid;
  unsigned* counter;
  unsigned* err;
  // down projection epilogue = AR_NORM
  float* resid;
  const float* gamma;
  float* xn_out;
  float eps;
  IhbComm comm;
} IhbMoeArgs;

int ihb_moe_gateup(IhbMoeArgs* args, int use_pdl, cudaStream_t stream);
int ihb_moe_down(IhbMoeArgs* args, int use_pdl, cudaStream_t stream);

// Embedding gather + first RMSNorm: resid = embed[*token]; xn = rmsnorm(resid) * gamma.
// xq / xs (optional): the normed vector again as a tensor-core activation row (e4m3 + scale per 128 channels when
// xq_fp8, else bf16).
int ihb_embed_norm(const void* embed, int embed_is_bf16, const int* token, int H, const float* gamma, float eps,
                   float* resid, float* xn, unsigned char* xq, float* xs, int xq_fp8, int use_pdl,
                   cudaStream_t stream);

// Per-head QK RMSNorm + NeoX RoPE at position *pos; writes q in place and K/V (bf16) into the cache row *pos.
// qkv: [(nq + 2 nkv) * 128] fp32 (Q heads, K heads, V heads); cos/sin: [max_seq, 64] fp32 tables.
int ihb_qk_norm_rope_kv(float* qkv, int nq, int nkv, const float* q_gamma, const float* k_gamma, float eps,
                        const float* cos_t, const float* sin_t, const int* pos, void* k_cache, void* v_cache,
                        int max_seq, int use_pdl, cudaStream_t stream);

// Split-KV GQA flash-decode over positions [0, *pos] with an in-kernel merge by the last CTA of each KV head.
// q: [nq, 128] fp32 (already normed + roped); k_cache/v_cache: [nkv, max_seq, 128] bf16; out: [nq, 128] fp32.
// out_q / out_s (optional): the output again as the o_proj kernel's activation row (one scale per head).
// scratch: nq * nsplit * 130 floats (partial acc, m, l); counters: nq unsigned, zero before the first launch.
int ihb_flash_decode(const float* q, const void* k_cache, const void* v_cache, int nq, int nkv, int max_seq,
                     const int* pos, int nsplit, float* scratch, unsigned* counters, float* out, unsigned char* out_q,
                     float* out_s, int out_fp8, int use_pdl, cudaStream_t stream);
size_t ihb_flash_decode_scratch_floats(int nq, int nsplit);
// The same two steps over an e4m3 KV cache: k_cache / v_cache [nkv, max_seq, 128] bytes, k_scale / v_scale
// [nkv, max_seq] fp32 (one scale per row = amax of the row / 448, written by the append; a row reads as byte * scale).
// The reference keeps its e4m3 cache with static per-channel scales (kernels/k1_attn_prologue.cu:524-604,
// kernels/k2_flash_decode.cu:71-83); the per-row scale needs no calibration pass.
int ihb_qk_norm_rope_kv8(float* qkv, int nq, int nkv, const float* q_gamma, const float* k_gamma, float eps,
                         const float* cos_t, const float* sin_t, const int* pos, void* k_cache, void* v_cache,
                         float* k_scale, float* v_scale, int max_seq, int use_pdl, cudaStream_t stream);
int ihb_flash_decode_kv8(const float* q, const void* k_cache, const void* v_cache, const float* k_scale,
                         const float* v_scale, int nq, int nkv, int max_seq, const int* pos, int nsplit, float* scratch,
                         unsigned* counters, float* out, unsigned char* out_q, float* out_s, int out_fp8, int use_pdl,
                         cudaStream_t stream);

// ---- tensor-core linear layers (tcgen05 / TMEM / TMA) ------------------------------------------------------------
enum { IHB_TC_LINEAR = 0, IHB_TC_GATEUP = 1, IHB_TC_DOWN = 2 };

// Y[t, r] = sum_k X[t, k] W[r, k] for T <= 128 tokens per call.
//   LINEAR: W [rows, K];            X [T_total, K];          out [T, out_stride] fp32
//   GATEUP: W [E][2][rows = I][K];  X [T_total, K];          out [top_k][T][I] = silu(gate) * up
//   DOWN:   W [E][rows = H][K = I]; X [top_k][T_total][K];   out [T, out_stride] = sum over slots of w_slot * (...)
// fp8: wscale [E][nrb][nkb_stride] (row blocks of rb rows, K blocks of 128), xscale [slots][nkb][T_total].
typedef struct {
  const void* W;
  const float* wscale;
  int wtype;               // IHB_W_FP8 | IHB_W_BF16 (activations have the same type)
  int rows, K;
  int rb, nrb, nkb_stride;
  int n_experts, expert0, top_k;
  const void* X;
  const float* xscale;
  int T, T_total, tok0;    // tokens in this call, rows of X, first token of this call
  int mode;
  const int* sel_idx;      // [top_k] global expert ids (GATEUP / DOWN)
  const float* sel_w;      // [top_k]
  float* out;
  int out_stride;
  float* partial;          // workspace of ihb_tc_partial_floats() floats when several units feed a tile
  unsigned* tile_counters; // one per output tile, zero before the first launch
  int ks, S, grid;         // K split / stages / CTAs (0 = choose)
  int n_units;             // filled in by the launcher
  unsigned* err;
  int tiled;               // 1: W is pre-tiled [matrix][k block][rows padded to 8][128 B] in swizzled order
  int x_rows1;             // 1 (needs tiled, T == 1): X is [slots][K padded to 128 B], one plain row per slot
  // Grouped mode (GATEUP / DOWN over tokens sorted by expert; top_k = 1, ks = 1): group g multiplies rows
  // [tok0, tok0 + ntok) of X (ntok <= the token tile) by local expert e. The table and its length live on the device,
  // so routing results never pass through the host. out rows are indexed by the sorted token position.
  const int* groups;       // [max_groups][4] = {e, tok0, ntok, 0}; NULL = not grouped
  const int* n_groups;     // device scalar
  int max_groups;
  // LINEAR over many tokens in ONE launch: tok_tiles > 1 tiles of tok_tile (16 / 32 / 64 / 128) tokens cover T tokens
  // (T may then exceed 128); every weight tile is then read from HBM once per launch instead of once per token tile
  int tok_tiles, tok_tile;
} IhbTcArgs;

int ihb_tc_gemm(IhbTcArgs* args, int use_pdl, cudaStream_t stream);
size_t ihb_tc_partial_floats(const IhbTcArgs* args);

// ---- single-token tensor-core linear layers with fused epilogues (the decode hot path) ----------------------------
enum { IHB_DEC_STORE = 0, IHB_DEC_AR_NORM = 1, IHB_DEC_ARGMAX = 2, IHB_DEC_ACT = 3 };

// y[r] = sum_k x[k] W[r, k] for ONE token. Weights are pre-tiled for HBM streaming:
//   W: [matrix][row tile][k block][rows of the tile, padded to 8][128 B], 16-byte chunks XOR-swizzled by row % 8
//   (matrix = expert, or expert * 2 + {gate, up}); a row tile's K blocks are contiguous, so one bulk copy moves
//   two of them (32 KB) into shared memory in the order the MMA descriptor expects.
//   X: [slots][k blocks * 128 B] plain activation rows (e4m3 or bf16), xscale [slots][k blocks] (e4m3 only).
// mode LINEAR + epi STORE / AR_NORM / ARGMAX; mode GATEUP + epi ACT (SwiGLU, then re-quantised per 128 rows as
// the down projection's input); mode DOWN + epi AR_NORM (sum over routing slots, weighted).
typedef struct {
  const void* W;
  const float* wscale;     // e4m3: [matrix rows / rb][nkb_stride] per expert: [E][nrb][nkb_stride]
  int wtype;
  int rows, K;
  int rb, nrb, nkb_stride;
  int n_experts, expert0, top_k;
  const void* X;
  const float* xscale;
  int mode, epi;
  const int* sel_idx;
  const float* sel_w;
  float* out;              // STORE: [rows] fp32; ARGMAX: optional logits [rows]
  unsigned char* act_q;    // ACT: [top_k][ceil(I * esize / 128) * 128 B]
  float* act_s;            // ACT (e4m3): [top_k][ceil(I / 128)]
  float* partial;          // ihb_tc_dec_partial_floats() floats (several units per output tile)
  unsigned* tile_counters; // one per output tile, zero before the first launch
  int ks, S, grid, n_units;
  unsigned* counter;       // last-CTA election (AR_NORM, ARGMAX), zero before the first launch
  unsigned* err;
  unsigned long long* argmax_partial;   // [grid]
  int vocab0;
  int* cur_token;
  int* pos;
  int* token_ring;
  int token_ring_size;
  const int* forced;
  const int* n_forced;
  float* resid;            // AR_NORM: as in IhbGemvArgs
  const float* gamma;
  float* xn_out;
  float eps;
  unsigned char* xq;       // AR_NORM: normed vector as the next tensor-core kernel's activation row (optional)
  float* xs;
  IhbComm comm;
} IhbTcDecArgs;

int ihb_tc_decode(IhbTcDecArgs* args, int use_pdl, cudaStream_t stream);
size_t ihb_tc_dec_partial_floats(const IhbTcDecArgs* args);

// ---- multi-token ("window") kernels: prompt chunks and speculative-verify windows -------------------------------------
// Row-wise RMSNorm (gamma != NULL) + activation quantisation: x [T][K] fp32 -> xn [T][K] fp32 (optional),
// xq [T][K] e4m3 (fp8 = 1, K % 128 == 0) or bf16, xs [K / 128][T] (fp8 only): the layout ihb_tc_gemm reads.
int ihb_norm_quant_rows(const float* x, const float* gamma, float eps, int K, int T, float* xn, unsigned char* xq,
                        float* xs, int fp8, cudaStream_t stream);
// qkv [T][(nq + 2 nkv) * 128] fp32: per-head RMSNorm + NeoX RoPE at positions[t]; q rows are rewritten in place, K / V
// rows go to cache row slots[t] (bf16).
int ihb_qk_norm_rope_rows(float* qkv, int nq, int nkv, const float* q_gamma, const float* k_gamma, float eps,
                          const float* cos_t, const float* sin_t, const int* positions, const int* slots, void* k_cache,
                          void* v_cache, int max_seq, int T, cudaStream_t stream);
// Query t (row t of qkv, qkv_stride floats apart) attends to cache rows [0, base) and to window row base + j when
// mask[t][j] != 0 (mask == NULL: causal, j <= t). out [T][nq * 128] fp32. mode 0: tensor-core tiles (16 tokens x 8
// heads per CTA, K / V blocks staged once for all of them); mode 1: one CTA per token on the CUDA cores.
// scratch (mode 0 only; may be NULL): ihb_window_attention_scratch_floats(nq, nkv, T) floats. With it, windows of few query
// tiles slice the keys over ihb_window_attention_splits(nq, nkv, base, T) CTAs per tile and a second kernel folds the
// slices' partial results; without it one CTA per tile walks all keys.
#define IHB_WINDOW_MAX_SPLITS 32
int ihb_window_attention(const float* qkv, int qkv_stride, const void* k_cache, const void* v_cache, int nq, int nkv,
                         int max_seq, int base, int T, const unsigned char* mask, float* out, int mode, float* scratch,
                         cudaStream_t stream);
int ihb_window_attention_splits(int nq, int nkv, int base, int T);
// The window append and the tensor-core tiles over an e4m3 KV cache (layout as for ihb_flash_decode_kv8). Rows are
// de-quantised on their way into shared memory; the tile loops are those of the bf16 cache.
int ihb_qk_norm_rope_rows_kv8(float* qkv, int nq, int nkv, const float* q_gamma, const float* k_gamma, float eps,
                              const float* cos_t, const float* sin_t, const int* positions, const int* slots, void* k_cache,
                              void* v_cache, float* k_scale, float* v_scale, int max_seq, int T, cudaStream_t stream);
int ihb_window_attention_kv8(const float* qkv, int qkv_stride, const void* k_cache, const void* v_cache, const float* k_scale,
                             const float* v_scale, int nq, int nkv, int max_seq, int base, int T, const unsigned char* mask,
                             float* out, float* scratch, cudaStream_t stream);
size_t ihb_window_attention_scratch_floats(int nq, int nkv, int T);

// ---- routing of a window of tokens on the device (moe_rows.cu) --------------------------------------------------------------------
// Fused router: logits = h W_r^T (h [T][H] fp32, router rows bf16 [E][H]), softmax, top-k with ties to the lowest id,
// optional renormalisation. logits (optional) [T][E], ti [T][top_k] global expert ids, tw [T][top_k]. E <= 256, top_k <= 8.
int ihb_router_topk_rows(const float* h, const void* router_bf16, int T, int H, int E, int top_k, int renorm, float* logits,
                         int* ti, float* tw, cudaStream_t stream);
// (token, slot) pairs bucketed by expert and cut into groups of at most nt rows: order [pairs] (pair at each sorted row),
// inv [pairs] (sorted row of each pair, -1 when its expert is not held here), groups [gmax][4] = {local expert, first
// row, rows, 0}, n_groups [1]. gmax >= E_local + pairs / nt + 1 holds every case.
int ihb_moe_group_table(const int* ti, int pairs, int expert0, int E_local, int nt, int* order, int* inv, int* groups,
                        int* n_groups, int gmax, cudaStream_t stream);
// out[p] = src[order[p] / k]: rows of row_bytes bytes (a multiple of 16) in expert order.
int ihb_moe_gather_rows(const void* src, const int* order, int k, int row_bytes, int pairs, void* out, cudaStream_t stream);
// y[t] = (resid ? resid[t] : 0) + sum over slots, in slot order, of tw[t][slot] * yg[inv[t k + slot]]  (rows of H floats).
int ihb_moe_combine_rows(const float* yg, const int* inv, const float* tw, int k, int H, int T, const float* resid, float* y,
                         cudaStream_t stream);

// Returns and clears the CUDA runtime's last-error word (a launch refused for its configuration leaves it set; the next
// entry point that ends in cudaGetLastError would report it as its own).
int ihb_clear_last_error(void);

// Block-scaled e4m3 weights W [nmat][rows][K] with scale [nmat][nrb][nkb] (one fp32 per rb x kb block) -> bf16 copies.
int ihb_dequant_bf16(const void* W, const float* scale, long long nmat, int rows, int K, int rb, int kb, int nrb, int nkb, void* out,
                     cudaStream_t stream);

// ---- stand-alone fused all-reduce (+ residual + RMSNorm) over symmetric memory -----------------------------------------
// x [T, H] fp32 partial of this rank -> out = sum over ranks (+ resid); out_norm = RMSNorm(out) * gamma (gamma != NULL);
// out_norm_bf16 (optional): the same normed rows rounded to bf16, the input format of the tensor-core GEMM that follows.
// algo 0 = by size, 1 = one-shot (push + one barrier, every rank adds), 2 = two-shot (row owners reduce with
// multimem.ld_reduce or peer loads and broadcast). Slot region (floats): one-shot 2 * nranks * T * H, two-shot
// 2 * T * H. counter: 8 unsigned words, zero before the first launch. One cooperative launch.
int ihb_allreduce_norm(const IhbComm* comm, const float* x, const float* resid, const float* gamma, float eps, int T,
                       int H, float* out, float* out_norm, void* out_norm_bf16, unsigned* counter, unsigned* err, int algo,
                       int grid, cudaStream_t stream);

// Latency-optimal all-reduce (+ residual + RMSNorm) of a few rows: one CTA per row, plain launch; every rank ADDS its row
// into 64-bit counted fixed-point slots on every GPU (multimem.red.add.u64 or peer reds) and waits for the contribution
// count on its own copy: one one-way trip through NVSwitch, no barrier. comm->slots_*: 4 * IHB_ARC_MAX_ROWS * H 64-bit
// words, zeroed before the first call and used by this entry only; call_counter: IHB_ARC_MAX_ROWS unsigned, zero at first
// (one call count per row, so calls with different T may follow each other; all ranks make the same calls); counter:
// unused. x fp32, or bf16 when x_is_bf16. T <= IHB_ARC_MAX_ROWS, H % 4 == 0, H <= 8192.
#define IHB_ARC_MAX_ROWS 64
int ihb_allreduce_counted(const IhbComm* comm, const void* x, int x_is_bf16, const float* resid, const float* gamma, float eps,
                          int T, int H, float* out, float* out_norm, void* out_norm_bf16, unsigned* counter,
                          unsigned* call_counter, unsigned* err, cudaStream_t stream);

// ---- all-to-all exchange of rows over peer memory (expert-parallel dispatch / combine for multi-token windows) -----
// Rows for destination d are pairs offsets[d] .. offsets[d + 1] of `send` (through `gather` when given). Receive region
// of every rank: [2 parities][nranks sources][cap rows][row_floats]; counts: [2][nranks] ints; flag: one arrival
// counter, zero before round 0. `round` is the number of exchanges made so far on this region (same on all ranks);
// all ranks pass the same grid. After the kernel, rows [0, counts[parity][s]) from source s are in place.
typedef struct {
  int nranks, rank;
  int row_floats;                            // multiple of 4
  int cap;
  unsigned round;
  const float* send;
  const int* gather;                         // optional [P]
  const int* offsets;                        // device, [nranks + 1]
  float* recv_peer[IHB_MAX_RANKS];
  int* count_peer[IHB_MAX_RANKS];
  unsigned* flag_peer[IHB_MAX_RANKS];
  unsigned* flag_local;
  unsigned* err;
} IhbA2AArgs;
int ihb_a2a_rows(const IhbA2AArgs* args, int grid, cudaStream_t stream);

// ---- persistent decode megakernel: one cooperative launch runs `steps` whole tokens -------------------------------------
// One weight matrix (or a stack of per-expert matrices with the same shape): rows contiguous, K-major.
typedef struct {
  const uint8_t* W;
  const float* wscale;     // fp8: [matrices][ceil(rows / rb)][nkb]
  int rows, K;             // per matrix
  int rb, kb_shift, nkb;   // scale block: rb rows x (16 << kb_shift) columns; nkb = floats per scale row
} IhbMat;

typedef struct {
  IhbMat wqkv;             // [(nq + 2 nkv) * 128, H]
  IhbMat wo;               // [H, nq * 128]
  IhbMat wgu;              // per expert [2 I, H] (gate rows then up rows)
  IhbMat wd;               // per expert [H, I]
  const void* router;      // bf16 [E, H]
  const float* in_ln;
  const float* post_ln;
  const float* q_norm;
  const float* k_norm;
  void* k_cache;           // [nkv, max_seq, 128] bf16
  void* v_cache;
  float* router_logits;    // [E] {fp32 value, tag} pairs (8 bytes each; zero-initialised)
  int* sel_idx;            // [top_k]
  float* sel_w;            // [top_k]
} IhbMegaLayer;

typedef struct {
  const IhbMegaLayer* layers;   // device array
  int n_layers;
  int wtype;                    // IHB_W_FP8 | IHB_W_BF16 (all linear layers; the router is always bf16)
  int H, nq, nkv, I, E, top_k, renorm;
  int expert0, E_local;         // experts held by this rank (expert parallel: a slice; tensor parallel: all, with I split)
  float attn_ar_scale;          // weight of the summed attention partials: tp / world (hybrid and pure expert
                                // parallel layouts compute the same attention shard on world / tp ranks)
  int max_seq;
  const float* cos_t;           // [max_seq, 64]
  const float* sin_t;
  float eps;
  const void* embed;            // [vocab, H] fp32 or bf16
  int embed_is_bf16;
  const float* final_norm;
  IhbMat lm_head;               // [vocab_local, H]
  int vocab0;
  float* logits;                // optional [vocab_local]
  int* cur_token;
  int* pos;
  int* token_ring;
  int token_ring_size;
  const int* forced;
  const int* n_forced;
  float* qkv;                   // [(nq + 2 nkv) * 128] {fp32 value, tag} pairs (8 bytes each; zero-initialised)
  float* attn_part;             // [nq][max_split][132]: partial records of the long-context attention mode
  float* attn;                  // [nq * 128] {value, tag} pairs: merged output of the long-context attention mode
  unsigned long long* attn_rec; // [nq][16][66] 8-byte words: per (head, block of 128 positions) 64 {half2, tag} pairs of the
                                // normalised partial output, {m, tag}, {l, tag}; merged by the CTAs that stage the
                                // o_proj input while nq * blocks <= 256 (NULL: always use the long-context mode)
  float* act;                   // [top_k * 2 I] {value, tag} pairs
  unsigned long long* argmax_partial;   // [grid]
  unsigned* bar;                // [0] grid-barrier arrivals, [2] their base for the next launch, [8 ...] attention merge counters
  unsigned* err;
  unsigned long long* prof;     // optional, 2 * prof_n words: CTA 0 stores %globaltimer at kernel start ([0]) and at the end of
                                // phase i ([i]); from [6 n_layers + 4]: per layer, start of the expert phase, selection done,
                                // gate/up done, activations seen. [prof_n + i]: the latest stamp of any CTA for phase i
                                // (atomic maximum: zero this half before a launch)
  int prof_n;
  int max_split;                // attention splits available per (kv head, group of 8 query heads) in the long-context mode
  int steps;                    // tokens per launch
  int ar_loopback;              // one rank only: k > 1 makes every all-reduce slot receive k adds (the traffic of k ranks)
  int delay_cta, delay_ns;      // test aid: CTA delay_cta idles delay_ns (at most 1 ms) before each of its all-reduce reads,
                                // so that a test can make one CTA of one GPU lag behind every other; delay_ns = 0: off
  IhbComm comm;
} IhbMegaArgs;

// grid = 0: one CTA per SM, at most H / 4 (every CTA must own rows of every all-reduce round). Returns
// cudaErrorCooperativeLaunchTooLarge when the CTAs cannot all be resident.
int ihb_mega_decode(const IhbMegaArgs* args, int grid, cudaStream_t stream);
int ihb_mega_max_grid(const IhbMegaArgs* args);

#ifdef __cplusplus
}
#endif
