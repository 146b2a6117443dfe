// C ABI of the host control plane (libihb_ctrl.so): speculative-decoding acceptance and cost models (spec.cpp),
// expert-routing placement / prediction / prefetch scheduling (routing.cpp). Everything is plain arrays and opaque
// handles so that Python (ctypes) and C++ callers share one implementation.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// ---- speculative decoding -------------------------------------------------------------------------------------------
// target_logits [(k + 1)][vocab]: row[pos] scores draft_tokens[pos]; row[k] is the bonus distribution.
// rng_u [k + 1]: u[pos] decides position pos, u[k] draws the correction / bonus token.
// Writes the emitted tokens (accepted prefix + one more) and returns their count.
int ihb_spec_accept(const float* target_logits, int vocab, int k, const int* draft_tokens, const float* draft_logprobs,
                    const float* rng_u, float temperature, int* out_tokens, int* out_n_accepted);

// As above with the drafter's full distributions draft_probs [k][vocab] (exactly lossless for sampling drafters).
int ihb_spec_accept_full(const float* target_logits, int vocab, int k, const int* draft_tokens, const float* draft_probs,
                         const float* rng_u, float temperature, int* out_tokens, int* out_n_accepted);

// n_drafters chains of k tokens; target_logits [n_drafters][k + 1][vocab]; rng_u needs n_drafters * k + 1 entries.
int ihb_spec_accept_multi(const float* target_logits, int vocab, int n_drafters, int k, const int* draft_tokens,
                          const float* draft_logprobs, const float* rng_u, float temperature, int* out_tokens,
                          int* out_n_accepted, int* winner, unsigned char* accept_mask);

// Token tree (node 0 = root sentinel); target_rows [n_nodes][vocab], row i scores node i's children.
int ihb_spec_accept_tree(int n_nodes, const int* tokens, const int* parent, const float* draft_logprob,
                         const float* target_rows, int vocab, const float* rng_u, int n_u, float temperature,
                         int* out_tokens, int* out_nodes, int* out_n_accepted);

int ihb_tree_attn_build(int n_nodes, const int* parent, int context_len, int* out_pos_id, int* out_anc_off,
                        int* out_anc_slots);
void ihb_tree_mask(int n_nodes, const int* parent, unsigned char* mask);

int ihb_draft_top_candidates(const int* d2t, const float* draft_logits, int draft_vocab, int m, int* out_tokens,
                             float* out_logprobs);

void ihb_sdpa_tree_ref(int n_nodes, const int* parent, int context_len, int n_q, int n_kv, int hd, const float* q,
                       const float* k_ctx, const float* v_ctx, const float* k_draft, const float* v_draft,
                       const float* q_gamma, const float* k_gamma, float eps, float theta, float* out);

// One chain round on the host: top-1 draft candidates from draft_logits [k][draft_vocab] -> verify(ctx, tokens, k,
// rows[(k + 1) * vocab]) -> accept. Returns the emitted count.
typedef void (*ihb_verify_fn)(void* ctx, const int* draft_tokens, int k, float* out_rows);
int ihb_spec_round(const int* d2t, const float* draft_logits, int draft_vocab, int k, int vocab, ihb_verify_fn verify,
                   void* verify_ctx, const float* rng_u, float temperature, int* out_tokens, int* out_n_accepted);

float ihb_verify_cost(unsigned union_size, float floor_fraction, float top_k);
int ihb_adaptive_verify_depth(const float* accept_probs, int k, const int* expert_off, const int* expert_ids,
                              float floor_fraction, float top_k, float* out_emitted, unsigned* out_union,
                              float* out_cost, float* out_value);
float ihb_level_advance_prob(float p, int branch);
float ihb_tree_expected_accepted(float first_pos, float p, int branch, int depth);
unsigned long long ihb_tree_nodes(int branch, int depth);
float ihb_persistence(float mean_accept_len, float first_pos, int depth);
float ihb_tree_shape_optimal(float mean_accept_len, float first_pos, float verify_flat_cost, float head_level_cost,
                             unsigned long long node_budget, int max_branch, int max_depth, int* out_branch,
                             int* out_depth, float* out_emitted);
float ihb_predict_speedup(float mean_accept_len, float first_pos, int depth, unsigned union_size, float floor_fraction,
                          float head_eager_cost, float draft_graph_cost, int graphs);
int ihb_route_aware_select(int n_cand, const float* draft_logprobs, const int* expert_off, const int* expert_ids,
                           const unsigned char* union_bits, float lambda);

// ---- routing ----------------------------------------------------------------------------------------------------------
enum { IHB_PREFETCH_WARM = 0, IHB_PREFETCH_DISPATCH = 1 };
typedef void (*ihb_prefetch_sink_fn)(void* ctx, int kind, int layer, int expert, int gpu);

void ihb_placement_optimize(const unsigned* counts, int n_layers, int n_experts, int n_gpus, double hot_mult,
                            int* out_primary, int* out_replica, double* out_stats);

void* ihb_pred_create(int n_layers, int hidden, int n_experts);
void ihb_pred_destroy(void* h);
void ihb_pred_set_router(void* h, int layer, const float* w);
void ihb_pred_linear_from_proxy(void* h);
void ihb_pred_linear_update(void* h, int layer, const float* hidden_batch, const float* target, int batch, float lr);
void ihb_pred_markov_enable(void* h);
void ihb_pred_markov_observe(void* h, int layer, const int* experts_l, int n_l, const int* experts_l1, int n_l1);
int ihb_pred_predict(void* h, int kind, int layer, const float* hidden, const int* cur_experts, int n_cur, int top_k,
                     const float* weights, int* out_ids, float* out_scores);

void* ihb_sched_create(int n_layers, int n_experts, int n_gpus, const int* primary, const int* replica);
void ihb_sched_destroy(void* h);
void ihb_sched_set_sink(void* h, ihb_prefetch_sink_fn fn, void* ctx, int record);
int ihb_sched_gpus_for(void* h, int layer, int expert, int* out_replica);
int ihb_sched_on_prediction(void* h, int layer, const int* experts, int n);
void ihb_sched_on_layer_complete(void* h, int layer, const int* actual, int n);
float ihb_sched_hit_rate(void* h);
unsigned long long ihb_sched_total_hits(void* h);
unsigned long long ihb_sched_total_prefetched(void* h);
int ihb_sched_drain(void* h, int* out, int cap);

void* ihb_acc_create(int n_layers, int top_k);
void ihb_acc_destroy(void* h);
void ihb_acc_record(void* h, int layer, const int* predicted, int n_pred, const int* actual, int n_actual);
float ihb_acc_hit_rate(void* h, int layer);
unsigned long long ihb_acc_tokens(void* h, int layer);
float ihb_acc_mean_hit_rate(void* h);
void ihb_acc_reset(void* h);

void* ihb_trace_create(int hidden, int n_experts, int max_traces);
void ihb_trace_destroy(void* h);
int ihb_trace_push(void* h, int layer, const float* hidden, const float* logits);
int ihb_trace_count(void* h, int layer);
int ihb_trace_drain_layer(void* h, int layer, float* out_hidden, float* out_logits);
void ihb_trace_clear(void* h);

#ifdef __cplusplus
}
#endif
