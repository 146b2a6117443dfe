// Speculative-decoding control plane (host C++, C ABI): lossless chain / multi-drafter / tree acceptance, tree
// attention index builder, draft-vocabulary candidate extraction, a CPU oracle for tree-masked attention, and the
// cost models that pick verify depth and tree shape.
//
// Behavioural contracts taken from the reference (engine/native/spec_accept.h:11-19, engine/src/spec/accept.rs,
// engine/src/spec/tree.rs, engine/native/tree_attn.h, engine/native/draft_vocab.h, engine/native/sdpa_tree_ref.h,
// engine/src/spec/{adaptive_verify,tree_shape,projection,route_aware}.rs):
//   * row[pos] of the verify logits scores draft[pos] (row 0 follows the last committed token), row[k] is a real
//     bonus distribution - every round verifies k + 1 rows, also for several drafters (the reference's
//     multi-drafter path substitutes a greedy stand-in on full accept, engine/src/spec/accept.rs:104-112);
//   * draft log-probabilities are in the draft head's own vocabulary space;
//   * acceptance is exact: u < min(1, p_target / p_draft), on rejection sample the residual max(0, p_t - p_d).
// `temperature <= 0` makes the target distribution the one-hot argmax (greedy decoding stays greedy).
#include "ctrl.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <numeric>
#include <vector>

namespace {

void softmax_row(const float* logits, int vocab, float temperature, std::vector<float>& p) {
  p.resize(vocab);
  if (temperature <= 0.f) {
    int best = 0;
    for (int i = 1; i < vocab; ++i)
      if (logits[i] > logits[best]) best = i;
    std::fill(p.begin(), p.end(), 0.f);
    p[best] = 1.f;
    return;
  }
  float mx = logits[0];
  for (int i = 1; i < vocab; ++i) mx = std::max(mx, logits[i]);
  double sum = 0.0;
  for (int i = 0; i < vocab; ++i) {
    p[i] = std::exp((logits[i] - mx) / temperature);
    sum += p[i];
  }
  const float inv = sum > 0.0 ? static_cast<float>(1.0 / sum) : 0.f;
  for (int i = 0; i < vocab; ++i) p[i] = sum > 0.0 ? p[i] * inv : 1.f / vocab;
}

int sample_from(const std::vector<float>& p, float u) {
  double total = 0.0;
  for (float v : p) total += v;
  if (total <= 0.0) return static_cast<int>(std::max_element(p.begin(), p.end()) - p.begin());
  const double t = static_cast<double>(u) * total;
  double cum = 0.0;
  int last = 0;
  for (size_t i = 0; i < p.size(); ++i) {
    if (p[i] <= 0.f) continue;
    cum += p[i];
    last = static_cast<int>(i);
    if (t < cum) return last;
  }
  return last;
}

// A drafted id outside the vocabulary (a drafter bug, a stale id map) has target probability 0: it is never accepted and
// never used as an index.
inline bool in_vocab(int x, int vocab) { return x >= 0 && x < vocab; }

// residual of target p against a drafter that put probability q on token x only
int sample_residual_point(const std::vector<float>& target, int x, float q, float u) {
  std::vector<float> p = target;
  if (in_vocab(x, static_cast<int>(p.size()))) p[x] = std::max(0.f, p[x] - q);
  double total = 0.0;
  for (float v : p) total += v;
  if (total < 1e-9) return sample_from(target, u);   // degenerate: the drafter's mass covers the target's (all of it on x)
  return sample_from(p, u);
}

// parent of node n for the tree walks below: an index that is not a node, or the node itself, counts as the root
inline int parent_of(const int* parent, int n, int n_nodes) {
  const int p = parent[n];
  return (p >= 0 && p < n_nodes && p != n) ? p : 0;
}

}  // namespace

extern "C" {

int ihb_spec_accept(const float* target_logits, int vocab, int k, const int* draft_tokens, const float* draft_logprobs,
                    const float* rng_u, float temperature, int* out_tokens, int* out_n_accepted) {
  std::vector<float> p;
  int accepted = 0;
  for (int pos = 0; pos < k; ++pos) {
    softmax_row(target_logits + static_cast<size_t>(pos) * vocab, vocab, temperature, p);
    const int x = draft_tokens[pos];
    const float q = std::exp(draft_logprobs[pos]);
    const float ratio = !in_vocab(x, vocab) ? 0.f : q > 0.f ? std::min(1.f, p[x] / q) : 1.f;
    if (rng_u[pos] < ratio) {
      out_tokens[accepted++] = x;
      continue;
    }
    out_tokens[accepted] = sample_residual_point(p, x, q, rng_u[k]);
    *out_n_accepted = accepted;
    return accepted + 1;
  }
  softmax_row(target_logits + static_cast<size_t>(k) * vocab, vocab, temperature, p);
  out_tokens[accepted] = sample_from(p, rng_u[k]);
  *out_n_accepted = accepted;
  return accepted + 1;
}

// Same walk with the drafter's FULL distribution per position (draft_probs [k][vocab]): the residual is
// max(0, p - q) over the whole vocabulary, which makes sampling drafters exactly lossless at any temperature.
int ihb_spec_accept_full(const float* target_logits, int vocab, int k, const int* draft_tokens, const float* draft_probs,
                         const float* rng_u, float temperature, int* out_tokens, int* out_n_accepted) {
  std::vector<float> p;
  int accepted = 0;
  for (int pos = 0; pos < k; ++pos) {
    softmax_row(target_logits + static_cast<size_t>(pos) * vocab, vocab, temperature, p);
    const float* q = draft_probs + static_cast<size_t>(pos) * vocab;
    const int x = draft_tokens[pos];
    const float ratio = !in_vocab(x, vocab) ? 0.f : q[x] > 0.f ? std::min(1.f, p[x] / q[x]) : 1.f;
    if (rng_u[pos] < ratio) {
      out_tokens[accepted++] = x;
      continue;
    }
    double total = 0.0;
    for (int i = 0; i < vocab; ++i) { p[i] = std::max(0.f, p[i] - q[i]); total += p[i]; }
    if (total < 1e-12) softmax_row(target_logits + static_cast<size_t>(pos) * vocab, vocab, temperature, p);
    out_tokens[accepted] = sample_from(p, rng_u[k]);
    *out_n_accepted = accepted;
    return accepted + 1;
  }
  softmax_row(target_logits + static_cast<size_t>(k) * vocab, vocab, temperature, p);
  out_tokens[accepted] = sample_from(p, rng_u[k]);
  *out_n_accepted = accepted;
  return accepted + 1;
}

// N drafters, each a chain of k tokens (row-major by drafter). target_logits: [n][k + 1][vocab] (drafter d's rows).
// Position by position the surviving drafters are tried in order; a drafter survives while its prefix equals the
// accepted prefix. Returns #emitted; *winner = drafter whose chain was followed last (-1: none).
int ihb_spec_accept_multi(const float* target_logits, int vocab, int n_drafters, int k, const int* draft_tokens,
                          const float* draft_logprobs, const float* rng_u, float temperature, int* out_tokens,
                          int* out_n_accepted, int* winner, unsigned char* accept_mask) {
  std::vector<float> p;
  std::vector<char> alive(n_drafters, 1);
  int accepted = 0, follow = 0, ui = 0;
  *winner = -1;
  if (accept_mask) std::memset(accept_mask, 0, static_cast<size_t>(n_drafters) * k);
  for (int pos = 0; pos < k; ++pos) {
    // all alive drafters share the accepted prefix, so any alive drafter's row[pos] is the same distribution
    int ref = -1;
    for (int d = 0; d < n_drafters; ++d)
      if (alive[d]) { ref = d; break; }
    if (ref < 0) break;
    softmax_row(target_logits + (static_cast<size_t>(ref) * (k + 1) + pos) * vocab, vocab, temperature, p);
    int taken = -1, best = ref;
    float best_ratio = -1.f;
    std::vector<float> resid = p;
    for (int d = 0; d < n_drafters && taken < 0; ++d) {
      if (!alive[d]) continue;
      const int x = draft_tokens[d * k + pos];
      const float q = std::exp(draft_logprobs[d * k + pos]);
      const bool ok = in_vocab(x, vocab);
      const float ratio = !ok ? 0.f : q > 0.f ? std::min(1.f, resid[x] / q) : 1.f;
      if (ratio > best_ratio) { best_ratio = ratio; best = d; }
      if (rng_u[ui++] < ratio) {
        taken = d;
      } else {                                   // SpecInfer-style: remove this drafter's mass, renormalise
        if (ok) resid[x] = std::max(0.f, resid[x] - q);
        double s = 0.0;
        for (float v : resid) s += v;
        if (s > 1e-12) for (float& v : resid) v = static_cast<float>(v / s);
      }
    }
    if (taken < 0) {
      out_tokens[accepted] = sample_from(resid, rng_u[ui++]);
      *out_n_accepted = accepted;
      if (*winner < 0) *winner = best;
      return accepted + 1;
    }
    const int tok = draft_tokens[taken * k + pos];
    out_tokens[accepted++] = tok;
    follow = taken;
    *winner = taken;
    if (accept_mask) accept_mask[taken * k + pos] = 1;
    for (int d = 0; d < n_drafters; ++d)
      if (alive[d] && draft_tokens[d * k + pos] != tok) alive[d] = 0;
  }
  softmax_row(target_logits + (static_cast<size_t>(follow) * (k + 1) + accepted) * vocab, vocab, temperature, p);
  out_tokens[accepted] = sample_from(p, rng_u[ui]);
  *out_n_accepted = accepted;
  return accepted + 1;
}

// Tree acceptance. Node 0 is the root sentinel (the last committed token); row[i] scores node i's children.
int ihb_spec_accept_tree(int n_nodes, const int* tokens, const int* parent, const float* draft_logprob,
                         const float* target_rows, int vocab, const float* rng_u, int n_u, float temperature,
                         int* out_tokens, int* out_nodes, int* out_n_accepted) {
  std::vector<std::vector<int>> kids(n_nodes);
  for (int i = 1; i < n_nodes; ++i)
    if (parent[i] >= 0 && parent[i] < n_nodes && parent[i] != i) kids[parent[i]].push_back(i);
  std::vector<float> p;
  int accepted = 0, node = 0, ui = 0;
  auto next_u = [&]() { return ui < n_u ? rng_u[ui++] : 0.5f; };
  for (;;) {
    softmax_row(target_rows + static_cast<size_t>(node) * vocab, vocab, temperature, p);
    auto order = kids[node];
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return draft_logprob[a] > draft_logprob[b]; });
    int go = -1;
    for (int c : order) {
      const int x = tokens[c];
      const float q = std::exp(draft_logprob[c]);
      const bool ok = in_vocab(x, vocab);
      const float a = !ok ? 0.f : q > 0.f ? std::min(1.f, p[x] / q) : 1.f;
      if (next_u() < a) { go = c; break; }
      if (ok) p[x] = std::max(0.f, p[x] - q);
      double s = 0.0;
      for (float v : p) s += v;
      if (s > 1e-12) for (float& v : p) v = static_cast<float>(v / s);
    }
    if (go < 0) {   // leaf, or every child rejected: sample what is left of the target distribution
      out_tokens[accepted] = sample_from(p, next_u());
      *out_n_accepted = accepted;
      return accepted + 1;
    }
    if (out_nodes) out_nodes[accepted] = go;
    out_tokens[accepted++] = tokens[go];
    node = go;
  }
}

// RoPE position and ancestor KV slots per node: node i > 0 lives in draft slot context_len + (i - 1); the root is
// the last committed token. Ancestors are listed root-side first, self last. Returns the slots written.
int ihb_tree_attn_build(int n_nodes, const int* parent, int context_len, int* out_pos_id, int* out_anc_off,
                        int* out_anc_slots) {
  int w = 0;
  out_anc_off[0] = 0;
  for (int i = 0; i < n_nodes; ++i) {
    // a walk of more than n_nodes steps means the parent array has a cycle: it is cut there
    int depth = 0;
    for (int n = i; n != 0 && depth < n_nodes; n = parent_of(parent, n, n_nodes)) ++depth;
    out_pos_id[i] = context_len + depth - 1;
    const int start = w;
    int steps = 0;
    for (int n = i; n != 0 && steps < depth; n = parent_of(parent, n, n_nodes), ++steps) out_anc_slots[w++] = context_len + (n - 1);
    std::reverse(out_anc_slots + start, out_anc_slots + w);
    out_anc_off[i + 1] = w;
  }
  return w;
}

// Boolean visibility [n_nodes - 1][n_nodes - 1] among the draft nodes (row = query node i + 1, column = key node
// j + 1): a node sees itself and its ancestors.
void ihb_tree_mask(int n_nodes, const int* parent, unsigned char* mask) {
  const int m = n_nodes - 1;
  std::memset(mask, 0, static_cast<size_t>(m) * m);
  for (int i = 1; i < n_nodes; ++i) {
    int steps = 0;
    for (int n = i; n != 0 && steps < n_nodes; n = parent_of(parent, n, n_nodes), ++steps)
      mask[static_cast<size_t>(i - 1) * m + (n - 1)] = 1;
  }
}

// Top-m draft candidates: target token ids through d2t, log-probabilities from the DRAFT-space log-softmax.
int ihb_draft_top_candidates(const int* d2t, const float* draft_logits, int draft_vocab, int m, int* out_tokens,
                             float* out_logprobs) {
  m = std::min(m, draft_vocab);
  float mx = draft_logits[0];
  for (int i = 1; i < draft_vocab; ++i) mx = std::max(mx, draft_logits[i]);
  double sum = 0.0;
  for (int i = 0; i < draft_vocab; ++i) sum += std::exp(draft_logits[i] - mx);
  const float lse = mx + static_cast<float>(std::log(sum));
  std::vector<int> idx(draft_vocab);
  std::iota(idx.begin(), idx.end(), 0);
  std::partial_sort(idx.begin(), idx.begin() + m, idx.end(), [&](int a, int b) {
    return draft_logits[a] > draft_logits[b] || (draft_logits[a] == draft_logits[b] && a < b);
  });
  for (int j = 0; j < m; ++j) {
    out_tokens[j] = d2t ? d2t[idx[j]] : idx[j];
    out_logprobs[j] = draft_logits[idx[j]] - lse;
  }
  return m;
}

// fp32 oracle of tree-masked GQA attention for one layer: per-head RMSNorm on q (and on the draft K rows), NeoX
// RoPE at pos_id, softmax over the committed context plus the node's ancestor draft slots.
//   q [n_nodes][n_q][hd] raw; k_ctx / v_ctx [n_kv][context_len][hd] (already normed + roped);
//   k_draft / v_draft [n_nodes][n_kv][hd] raw (node 0 unused); out [n_nodes][n_q][hd] (node 0 left zero).
void ihb_sdpa_tree_ref(int n_nodes, const int* parent, int context_len, int n_q, int n_kv, int hd, const float* q,
                       const float* k_ctx, const float* v_ctx, const float* k_draft, const float* v_draft,
                       const float* q_gamma, const float* k_gamma, float eps, float theta, float* out) {
  std::vector<int> pos(n_nodes), off(n_nodes + 1), slots(static_cast<size_t>(n_nodes) * n_nodes + 1);
  ihb_tree_attn_build(n_nodes, parent, context_len, pos.data(), off.data(), slots.data());
  const int half = hd / 2, g = n_q / n_kv;
  auto norm_rope = [&](const float* x, const float* gamma, int position, float* y) {
    double ss = 0.0;
    for (int d = 0; d < hd; ++d) ss += static_cast<double>(x[d]) * x[d];
    const float rinv = 1.f / std::sqrt(static_cast<float>(ss / hd) + eps);
    std::vector<float> t(hd);
    for (int d = 0; d < hd; ++d) t[d] = x[d] * rinv * gamma[d];
    for (int d = 0; d < half; ++d) {
      const float ang = position * std::pow(theta, -static_cast<float>(d) / half);
      const float c = std::cos(ang), s = std::sin(ang);
      y[d] = t[d] * c - t[d + half] * s;
      y[d + half] = t[d + half] * c + t[d] * s;
    }
  };
  std::vector<float> kd(static_cast<size_t>(n_nodes) * n_kv * hd, 0.f);
  for (int i = 1; i < n_nodes; ++i)
    for (int h = 0; h < n_kv; ++h)
      norm_rope(k_draft + (static_cast<size_t>(i) * n_kv + h) * hd, k_gamma, pos[i], &kd[(static_cast<size_t>(i) * n_kv + h) * hd]);
  std::memset(out, 0, sizeof(float) * static_cast<size_t>(n_nodes) * n_q * hd);
  const float scale = 1.f / std::sqrt(static_cast<float>(hd));
  std::vector<float> qr(hd), sc;
  for (int i = 1; i < n_nodes; ++i) {
    for (int h = 0; h < n_q; ++h) {
      const int kvh = h / g;
      norm_rope(q + (static_cast<size_t>(i) * n_q + h) * hd, q_gamma, pos[i], qr.data());
      const int n_anc = off[i + 1] - off[i];
      sc.assign(context_len + n_anc, 0.f);
      for (int t = 0; t < context_len; ++t) {
        const float* kr = k_ctx + (static_cast<size_t>(kvh) * context_len + t) * hd;
        float s = 0.f;
        for (int d = 0; d < hd; ++d) s += qr[d] * kr[d];
        sc[t] = s * scale;
      }
      for (int a = 0; a < n_anc; ++a) {
        const int node = slots[off[i] + a] - context_len + 1;
        const float* kr = &kd[(static_cast<size_t>(node) * n_kv + kvh) * hd];
        float s = 0.f;
        for (int d = 0; d < hd; ++d) s += qr[d] * kr[d];
        sc[context_len + a] = s * scale;
      }
      float mx = sc[0];
      for (float v : sc) mx = std::max(mx, v);
      double sum = 0.0;
      for (float& v : sc) { v = std::exp(v - mx); sum += v; }
      float* o = out + (static_cast<size_t>(i) * n_q + h) * hd;
      for (int t = 0; t < context_len; ++t) {
        const float w = static_cast<float>(sc[t] / sum);
        const float* vr = v_ctx + (static_cast<size_t>(kvh) * context_len + t) * hd;
        for (int d = 0; d < hd; ++d) o[d] += w * vr[d];
      }
      for (int a = 0; a < n_anc; ++a) {
        const int node = slots[off[i] + a] - context_len + 1;
        const float w = static_cast<float>(sc[context_len + a] / sum);
        const float* vr = v_draft + (static_cast<size_t>(node) * n_kv + kvh) * hd;
        for (int d = 0; d < hd; ++d) o[d] += w * vr[d];
      }
    }
  }
}

int ihb_spec_round(const int* d2t, const float* draft_logits, int draft_vocab, int k, int vocab, ihb_verify_fn verify,
                   void* verify_ctx, const float* rng_u, float temperature, int* out_tokens, int* out_n_accepted) {
  std::vector<int> toks(k);
  std::vector<float> lps(k);
  for (int i = 0; i < k; ++i)
    ihb_draft_top_candidates(d2t, draft_logits + static_cast<size_t>(i) * draft_vocab, draft_vocab, 1, &toks[i], &lps[i]);
  std::vector<float> rows(static_cast<size_t>(k + 1) * vocab);
  verify(verify_ctx, toks.data(), k, rows.data());
  return ihb_spec_accept(rows.data(), vocab, k, toks.data(), lps.data(), rng_u, temperature, out_tokens, out_n_accepted);
}

// ---- cost models -------------------------------------------------------------------------------------------------
float ihb_verify_cost(unsigned union_size, float floor_fraction, float top_k) {
  const float f = std::min(1.f, std::max(0.f, floor_fraction));
  return f + (1.f - f) * (0.34f + 0.66f * static_cast<float>(union_size) / top_k);
}

static float expected_accepted(const float* probs, int n) {
  float total = 0.f, prefix = 1.f;
  for (int i = 0; i < n; ++i) {
    prefix *= std::min(1.f, std::max(0.f, probs[i]));
    total += prefix;
  }
  return total;
}

// Depth maximising emitted / verify cost; experts of position i are expert_ids[expert_off[i] .. expert_off[i+1]).
// Ties keep the shallower depth. Returns the depth (0 when there is nothing to verify).
int ihb_adaptive_verify_depth(const float* accept_probs, int k, const int* expert_off, const int* expert_ids,
                              float floor_fraction, float top_k, float* out_emitted, unsigned* out_union,
                              float* out_cost, float* out_value) {
  std::vector<char> seen(4096, 0);
  unsigned uni = 0;
  int best_d = 0;
  float best_v = -1.f;
  for (int d = 1; d <= k; ++d) {
    for (int e = expert_off[d - 1]; e < expert_off[d]; ++e) {
      const int id = expert_ids[e] & 4095;
      if (!seen[id]) { seen[id] = 1; ++uni; }
    }
    const float em = 1.f + expected_accepted(accept_probs, d);
    const float cost = ihb_verify_cost(uni, floor_fraction, top_k);
    const float value = cost > 0.f ? em / cost : INFINITY;
    if (value > best_v) {
      best_v = value; best_d = d;
      if (out_emitted) *out_emitted = em;
      if (out_union) *out_union = uni;
      if (out_cost) *out_cost = cost;
      if (out_value) *out_value = value;
    }
  }
  return best_d;
}

float ihb_level_advance_prob(float p, int branch) {
  p = std::min(1.f, std::max(0.f, p));
  return branch <= 0 ? 0.f : 1.f - std::pow(1.f - p, static_cast<float>(branch));
}

float ihb_tree_expected_accepted(float first_pos, float p, int branch, int depth) {
  float total = 0.f, prefix = 1.f;
  for (int i = 0; i < depth; ++i) {
    prefix *= ihb_level_advance_prob(i == 0 ? first_pos : p, branch);
    total += prefix;
  }
  return total;
}

unsigned long long ihb_tree_nodes(int branch, int depth) {
  unsigned long long total = 0, level = 1;
  for (int i = 0; i < depth; ++i) {
    level *= static_cast<unsigned long long>(branch);
    total += level;
  }
  return total;
}

// Per-position continuation probability that reproduces a measured mean accept length (bisection).
float ihb_persistence(float mean_accept_len, float first_pos, int depth) {
  const float target = std::max(0.f, mean_accept_len - 1.f);
  if (depth == 0 || first_pos <= 0.f) return 0.f;
  auto acc_at = [&](float p) {
    std::vector<float> probs(depth, p);
    probs[0] = std::min(1.f, std::max(0.f, first_pos));
    return expected_accepted(probs.data(), depth);
  };
  if (acc_at(0.f) >= target) return 0.f;
  float lo = 0.f, hi = 0.999f;
  if (acc_at(hi) < target) return hi;
  for (int i = 0; i < 40; ++i) {
    const float mid = 0.5f * (lo + hi);
    (acc_at(mid) < target ? lo : hi) = mid;
  }
  return 0.5f * (lo + hi);
}

// Best (branch, depth) under a node budget for cost = depth * head_level_cost + verify_flat_cost.
float ihb_tree_shape_optimal(float mean_accept_len, float first_pos, float verify_flat_cost, float head_level_cost,
                             unsigned long long node_budget, int max_branch, int max_depth, int* out_branch,
                             int* out_depth, float* out_emitted) {
  float best = -1.f;
  for (int b = 1; b <= std::max(1, max_branch); ++b) {
    for (int d = 1; d <= std::max(1, max_depth); ++d) {
      if (!(b == 1 && d == 1) && ihb_tree_nodes(b, d) > node_budget) continue;
      const float p = ihb_persistence(mean_accept_len, first_pos, d);
      const float em = 1.f + ihb_tree_expected_accepted(first_pos, p, b, d);
      const float cost = d * head_level_cost + verify_flat_cost;
      const float sp = cost > 0.f ? em / cost : 0.f;
      if (sp > best) {
        best = sp;
        *out_branch = b; *out_depth = d;
        if (out_emitted) *out_emitted = em;
      }
    }
  }
  return best;
}

// Speed-up predicted for a chain of `depth` drafts with measured acceptance, given the union of experts the verify
// pass lights up; graphs: the draft costs draft_graph_cost once instead of depth * head_eager_cost.
float ihb_predict_speedup(float mean_accept_len, float first_pos, int depth, unsigned union_size, float floor_fraction,
                          float head_eager_cost, float draft_graph_cost, int graphs) {
  const float p = ihb_persistence(mean_accept_len, first_pos, depth);
  std::vector<float> probs(std::max(depth, 1), p);
  probs[0] = std::min(1.f, std::max(0.f, first_pos));
  const float em = 1.f + expected_accepted(probs.data(), depth);
  const float round = (graphs ? draft_graph_cost : depth * head_eager_cost) + ihb_verify_cost(union_size, floor_fraction, 8.f);
  return round > 0.f ? em / round : INFINITY;
}

// Route-aware candidate choice: score = draft log-prob + lambda * |experts(c) ∩ union| ; returns the index.
int ihb_route_aware_select(int n_cand, const float* draft_logprobs, const int* expert_off, const int* expert_ids,
                           const unsigned char* union_bits /* 4096-bit set */, float lambda) {
  int best = -1;
  float best_score = -INFINITY;
  for (int c = 0; c < n_cand; ++c) {
    int overlap = 0;
    for (int e = expert_off[c]; e < expert_off[c + 1]; ++e) {
      const int id = expert_ids[e] & 4095;
      overlap += (union_bits[id >> 3] >> (id & 7)) & 1;
    }
    const float s = draft_logprobs[c] + lambda * overlap;
    if (s > best_score) { best_score = s; best = c; }
  }
  return best;
}

}  // extern "C"
