// Expert-routing control plane (host C++, C ABI): load-balanced expert placement with hot-expert replication,
// next-layer route predictors (router proxy, learned linear map, Markov transitions, score-fusion ensemble), the
// prefetch scheduler that turns predictions into warm / early-dispatch actions, and accuracy / trace bookkeeping.
//
// Same behaviour as the reference's engine/src/routing/{optimizer,predictor,scheduler,stats}.rs, exposed as opaque
// handles over flat arrays so that the Python engine and the CUDA sinks share one implementation.
#include "ctrl.h"

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <deque>
#include <numeric>
#include <vector>

namespace {
// expert ids wrap into [0, n) the way the placement lookups of the Python side do (id % n), negatives included:
// a stray id must never index outside a table
inline size_t wrap_id(int id, int n) {
  const int m = id % n;
  return static_cast<size_t>(m < 0 ? m + n : m);
}


float dotf(const float* a, const float* b, int n) {
  float s = 0.f;
  for (int i = 0; i < n; ++i) s += a[i] * b[i];
  return s;
}

int topk(const std::vector<float>& scores, int k, int* ids, float* vals) {
  k = std::min<int>(k, static_cast<int>(scores.size()));
  if (k <= 0) return 0;
  std::vector<int> idx(scores.size());
  std::iota(idx.begin(), idx.end(), 0);
  std::partial_sort(idx.begin(), idx.begin() + k, idx.end(),
                    [&](int a, int b) { return scores[a] > scores[b] || (scores[a] == scores[b] && a < b); });
  for (int j = 0; j < k; ++j) {
    ids[j] = idx[j];
    if (vals) vals[j] = scores[idx[j]];
  }
  return k;
}

struct Predictor {
  int n_layers, hidden, n_experts;
  std::vector<std::vector<float>> router;   // [layer][expert][hidden]; empty = not loaded
  std::vector<std::vector<float>> linear;   // [layer][expert][hidden] maps h_L to scores of layer L + 1
  std::vector<std::vector<float>> markov;   // [layer][from][to] counts, Laplace prior 1
  bool has_linear = false, has_markov = false;

  bool proxy_scores(int layer, const float* h, std::vector<float>& s) const {
    if (layer + 1 >= n_layers || router[layer + 1].empty()) return false;
    s.resize(n_experts);
    for (int e = 0; e < n_experts; ++e) s[e] = dotf(h, &router[layer + 1][static_cast<size_t>(e) * hidden], hidden);
    return true;
  }
  bool linear_scores(int layer, const float* h, std::vector<float>& s) const {
    if (!has_linear || layer + 1 >= n_layers || linear[layer].empty()) return false;
    s.resize(n_experts);
    for (int e = 0; e < n_experts; ++e) s[e] = dotf(h, &linear[layer][static_cast<size_t>(e) * hidden], hidden);
    return true;
  }
  bool markov_scores(int layer, const int* cur, int n_cur, std::vector<float>& s) const {
    if (!has_markov || layer < 0 || layer + 1 >= n_layers || cur == nullptr || n_cur <= 0) return false;
    s.assign(n_experts, 0.f);
    for (int i = 0; i < n_cur; ++i) {
      const float* row = &markov[layer][wrap_id(cur[i], n_experts) * n_experts];
      float sum = 0.f;
      for (int j = 0; j < n_experts; ++j) sum += row[j];
      for (int j = 0; j < n_experts; ++j) s[j] += row[j] / sum;
    }
    return true;
  }
};

struct Action { int kind, layer, expert, gpu; };

struct Scheduler {
  int n_layers, n_experts, n_gpus;
  std::vector<int> primary, replica;        // [layer][expert]; replica -1 = none
  struct Pending { int layer; std::vector<int> experts; };
  std::deque<Pending> pending;
  std::vector<Action> recorded;
  ihb_prefetch_sink_fn sink = nullptr;
  void* sink_ctx = nullptr;
  bool record = true;
  uint64_t prefetched = 0, hits = 0;
  void submit(const Action& a) {
    if (sink) sink(sink_ctx, a.kind, a.layer, a.expert, a.gpu);
    if (record) recorded.push_back(a);
  }
};

struct Accuracy {
  int n_layers, top_k;
  std::vector<uint64_t> hits, total;
};

struct Traces {
  int hidden, n_experts, max_traces;
  std::vector<float> h, logits;
  std::vector<int> layers;
};

double imbalance_of(const std::vector<double>& load) {
  double total = 0.0, mx = 0.0;
  for (double l : load) { total += l; mx = std::max(mx, l); }
  return total == 0.0 ? 1.0 : mx / (total / load.size());
}

}  // namespace

// helpers of the placement optimiser (see ihb_placement_optimize)
namespace {
struct Candidate {
  std::vector<int> prim, rep;
  double peak = 0.0;
};

double peak_of(const unsigned* c, int n_experts, int n_gpus, const std::vector<int>& prim, const std::vector<int>& rep,
               std::vector<double>* loads) {
  std::vector<double> load(n_gpus, 0.0);
  for (int e = 0; e < n_experts; ++e) {
    if (rep[e] >= 0) { load[prim[e]] += 0.5 * c[e]; load[rep[e]] += 0.5 * c[e]; }
    else load[prim[e]] += c[e];
  }
  if (loads != nullptr) *loads = load;
  return *std::max_element(load.begin(), load.end());
}

Candidate place_lpt(const unsigned* c, int n_experts, int n_gpus, const std::vector<char>& hot) {
  struct Item { double w; int e; };
  std::vector<Item> items;
  for (int e = 0; e < n_experts; ++e) {
    if (hot[e]) { items.push_back({0.5 * c[e], e}); items.push_back({0.5 * c[e], e}); }
    else items.push_back({static_cast<double>(c[e]), e});
  }
  std::stable_sort(items.begin(), items.end(), [](const Item& a, const Item& b) { return a.w > b.w; });
  Candidate out;
  out.prim.assign(n_experts, -1);
  out.rep.assign(n_experts, -1);
  std::vector<double> load(n_gpus, 0.0);
  for (const Item& it : items) {
    int best = -1;
    for (int g = 0; g < n_gpus; ++g) {
      if (g == out.prim[it.e]) continue;                 // the second half of a hot expert goes to another GPU
      if (best < 0 || load[g] < load[best]) best = g;
    }
    if (out.prim[it.e] < 0) out.prim[it.e] = best; else out.rep[it.e] = best;
    load[best] += it.w;
  }
  out.peak = peak_of(c, n_experts, n_gpus, out.prim, out.rep, nullptr);
  return out;
}
}  // namespace

extern "C" {

// ---- placement -------------------------------------------------------------------------------------------------------
// counts [n_layers][n_experts]; out_primary / out_replica [n_layers][n_experts] (replica -1 = none);
// out_stats = {round-robin mean imbalance, optimised mean imbalance, improvement %, replicated expert-layers}.
//
// Per layer three candidate placements are built and the one with the lowest peak load is kept:
//  (a) longest-processing-time: heaviest expert first onto the least-loaded GPU, no replicas;
//  (b) the same with every hot expert (count > hot_mult x the layer mean) split into two halves that are placed as
//      separate items on two different GPUs (primary = home of the first half, replica = home of the second), so a
//      replica is PLACED by load like any other item instead of being bolted on afterwards;
//  (c) round robin (expert % n_gpus), the layout to beat.
// Ties go to (b), then (a): a layer never ends up with a higher peak than round robin, and never with a replica that
// raises its peak. (The reference places by (a) and then always gives a hot expert a replica on the least-loaded other
// GPU, engine/src/routing/optimizer.rs:61-232; on skewed counts that step can undo the balance (a) had reached.)
void ihb_placement_optimize(const unsigned* counts, int n_layers, int n_experts, int n_gpus, double hot_mult,
                            int* out_primary, int* out_replica, double* out_stats) {
  double rr_total = 0.0, opt_total = 0.0;
  long replicated = 0;
  for (int l = 0; l < n_layers; ++l) {
    const unsigned* c = counts + static_cast<size_t>(l) * n_experts;
    int* prim = out_primary + static_cast<size_t>(l) * n_experts;
    int* rep = out_replica + static_cast<size_t>(l) * n_experts;
    Candidate rr;
    rr.prim.resize(n_experts);
    rr.rep.assign(n_experts, -1);
    for (int e = 0; e < n_experts; ++e) rr.prim[e] = e % n_gpus;
    std::vector<double> rr_load;
    rr.peak = peak_of(c, n_experts, n_gpus, rr.prim, rr.rep, &rr_load);
    rr_total += imbalance_of(rr_load);

    uint64_t total = 0;
    for (int e = 0; e < n_experts; ++e) total += c[e];
    std::vector<char> none(n_experts, 0), hot(n_experts, 0);
    bool any_hot = false;
    if (total > 0 && n_gpus > 1) {
      const double threshold = hot_mult * (static_cast<double>(total) / n_experts);
      for (int e = 0; e < n_experts; ++e) {
        hot[e] = static_cast<double>(c[e]) > threshold;
        any_hot = any_hot || hot[e];
      }
    }
    Candidate best = place_lpt(c, n_experts, n_gpus, none);
    if (any_hot) {
      Candidate split = place_lpt(c, n_experts, n_gpus, hot);
      if (split.peak <= best.peak) best = split;
    }
    if (rr.peak < best.peak) best = rr;
    std::vector<double> opt;
    peak_of(c, n_experts, n_gpus, best.prim, best.rep, &opt);
    opt_total += imbalance_of(opt);
    for (int e = 0; e < n_experts; ++e) {
      prim[e] = best.prim[e];
      rep[e] = best.rep[e];
      replicated += rep[e] >= 0;
    }
  }
  const double mean_rr = n_layers ? rr_total / n_layers : 1.0, mean_opt = n_layers ? opt_total / n_layers : 1.0;
  out_stats[0] = mean_rr;
  out_stats[1] = mean_opt;
  out_stats[2] = (1.0 - mean_opt / mean_rr) * 100.0;
  out_stats[3] = static_cast<double>(replicated);
}

// ---- predictors ------------------------------------------------------------------------------------------------------
void* ihb_pred_create(int n_layers, int hidden, int n_experts) {
  auto* p = new Predictor{n_layers, hidden, n_experts, {}, {}, {}};
  p->router.resize(n_layers);
  p->linear.resize(n_layers);
  return p;
}
void ihb_pred_destroy(void* h) { delete static_cast<Predictor*>(h); }

void ihb_pred_set_router(void* h, int layer, const float* w) {
  auto* p = static_cast<Predictor*>(h);
  if (layer < 0 || layer >= p->n_layers) return;
  p->router[layer].assign(w, w + static_cast<size_t>(p->n_experts) * p->hidden);
}

// P_L starts as the router of layer L + 1 (the residual stream changes little from one layer to the next)
void ihb_pred_linear_from_proxy(void* h) {
  auto* p = static_cast<Predictor*>(h);
  for (int l = 0; l + 1 < p->n_layers; ++l) p->linear[l] = p->router[l + 1];
  p->has_linear = true;
}

// one SGD step on mean squared error between h @ P_L^T and the observed next-layer router logits
void ihb_pred_linear_update(void* h, int layer, const float* hidden_batch, const float* target, int batch, float lr) {
  auto* p = static_cast<Predictor*>(h);
  if (!p->has_linear || layer < 0 || layer + 1 >= p->n_layers || p->linear[layer].empty()) return;
  const int hs = p->hidden, ne = p->n_experts;
  for (int e = 0; e < ne; ++e) {
    float* w = &p->linear[layer][static_cast<size_t>(e) * hs];
    for (int b = 0; b < batch; ++b) {
      const float* hb = hidden_batch + static_cast<size_t>(b) * hs;
      const float err = (dotf(hb, w, hs) - target[static_cast<size_t>(b) * ne + e]) / batch;
      for (int i = 0; i < hs; ++i) w[i] -= lr * err * hb[i];
    }
  }
}

void ihb_pred_markov_enable(void* h) {
  auto* p = static_cast<Predictor*>(h);
  p->markov.assign(std::max(0, p->n_layers - 1), std::vector<float>(static_cast<size_t>(p->n_experts) * p->n_experts, 1.f));
  p->has_markov = true;
}

void ihb_pred_markov_observe(void* h, int layer, const int* experts_l, int n_l, const int* experts_l1, int n_l1) {
  auto* p = static_cast<Predictor*>(h);
  if (!p->has_markov || layer < 0 || layer + 1 >= p->n_layers) return;
  for (int i = 0; i < n_l; ++i)
    for (int j = 0; j < n_l1; ++j)
      p->markov[layer][wrap_id(experts_l[i], p->n_experts) * p->n_experts + wrap_id(experts_l1[j], p->n_experts)] += 1.f;
}

// kind: 0 proxy, 1 learned linear, 2 Markov, 3 ensemble (weights[3], each component L2-normalised before mixing).
// Predicts the experts of layer `layer + 1`; returns how many ids were written (0 past the last layer).
int ihb_pred_predict(void* h, int kind, int layer, const float* hidden, const int* cur_experts, int n_cur, int top_k,
                     const float* weights, int* out_ids, float* out_scores) {
  auto* p = static_cast<Predictor*>(h);
  if (layer < 0 || layer + 1 >= p->n_layers) return 0;
  std::vector<float> s;
  if (kind == 0) {
    if (!p->proxy_scores(layer, hidden, s)) return 0;
  } else if (kind == 1) {
    if (!p->linear_scores(layer, hidden, s)) return 0;
  } else if (kind == 2) {
    if (!p->markov_scores(layer, cur_experts, n_cur, s)) return 0;
  } else {
    std::vector<float> fused(p->n_experts, 0.f), part;
    float total_w = 0.f;
    for (int c = 0; c < 3; ++c) {
      const float w = weights ? weights[c] : (c == 0 ? 1.f : 0.f);
      if (w <= 0.f) continue;
      const bool ok = c == 0 ? (hidden && p->proxy_scores(layer, hidden, part))
                    : c == 1 ? (hidden && p->linear_scores(layer, hidden, part))
                             : p->markov_scores(layer, cur_experts, n_cur, part);
      if (!ok) continue;
      float norm = 0.f;
      for (float v : part) norm += v * v;
      norm = std::max(std::sqrt(norm), 1e-9f);
      for (int e = 0; e < p->n_experts; ++e) fused[e] += w * part[e] / norm;
      total_w += w;
    }
    if (total_w <= 0.f) return 0;
    for (float& v : fused) v /= total_w;
    s.swap(fused);
  }
  return topk(s, top_k, out_ids, out_scores);
}

// ---- prefetch scheduler ----------------------------------------------------------------------------------------------
void* ihb_sched_create(int n_layers, int n_experts, int n_gpus, const int* primary, const int* replica) {
  auto* s = new Scheduler{n_layers, n_experts, n_gpus, {}, {}, {}, {}};
  const size_t n = static_cast<size_t>(n_layers) * n_experts;
  s->primary.resize(n);
  s->replica.assign(n, -1);
  for (size_t i = 0; i < n; ++i) s->primary[i] = primary ? primary[i] : static_cast<int>(i % n_experts) % n_gpus;
  if (replica) std::copy(replica, replica + n, s->replica.begin());
  return s;
}
void ihb_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }

void ihb_sched_set_sink(void* h, ihb_prefetch_sink_fn fn, void* ctx, int record) {
  auto* s = static_cast<Scheduler*>(h);
  s->sink = fn; s->sink_ctx = ctx; s->record = record != 0;
}

int ihb_sched_gpus_for(void* h, int layer, int expert, int* out_replica) {
  auto* s = static_cast<Scheduler*>(h);
  if (layer < 0 || layer >= s->n_layers) {
    if (out_replica) *out_replica = -1;
    return -1;
  }
  const size_t i = static_cast<size_t>(layer) * s->n_experts + wrap_id(expert, s->n_experts);
  if (out_replica) *out_replica = s->replica[i];
  return s->primary[i];
}

// A prediction for `layer` arrived: warm + early-dispatch every predicted expert on each GPU that hosts it.
int ihb_sched_on_prediction(void* h, int layer, const int* experts, int n) {
  auto* s = static_cast<Scheduler*>(h);
  if (layer < 0 || layer >= s->n_layers) return 0;
  int issued = 0;
  for (int i = 0; i < n; ++i) {
    const size_t at = static_cast<size_t>(layer) * s->n_experts + wrap_id(experts[i], s->n_experts);
    const int homes[2] = {s->primary[at], s->replica[at]};
    for (int g : homes) {
      if (g < 0) continue;
      s->submit({IHB_PREFETCH_WARM, layer, experts[i], g});
      s->submit({IHB_PREFETCH_DISPATCH, layer, experts[i], g});
      issued += 2;
    }
  }
  s->prefetched += n;
  s->pending.push_back({layer, std::vector<int>(experts, experts + n)});
  while (s->pending.size() > 4 * static_cast<size_t>(s->n_layers) + 4) s->pending.pop_front();   // never grows without bound
  return issued;
}

void ihb_sched_on_layer_complete(void* h, int layer, const int* actual, int n) {
  auto* s = static_cast<Scheduler*>(h);
  // score the oldest pending prediction for this layer; predictions queued before it were for layers whose routing
  // never arrived (a skipped layer, a stream that restarted): they stay counted as prefetched and are dropped
  auto it = std::find_if(s->pending.begin(), s->pending.end(), [layer](const auto& p) { return p.layer == layer; });
  if (it == s->pending.end()) return;
  for (int e : it->experts)
    if (std::find(actual, actual + n, e) != actual + n) ++s->hits;
  s->pending.erase(s->pending.begin(), it + 1);
}

float ihb_sched_hit_rate(void* h) {
  auto* s = static_cast<Scheduler*>(h);
  return s->prefetched ? static_cast<float>(s->hits) / static_cast<float>(s->prefetched) : 0.f;
}
unsigned long long ihb_sched_total_hits(void* h) { return static_cast<Scheduler*>(h)->hits; }
unsigned long long ihb_sched_total_prefetched(void* h) { return static_cast<Scheduler*>(h)->prefetched; }

// moves up to `cap` recorded actions (4 ints each: kind, layer, expert, gpu) into `out`; returns the count
int ihb_sched_drain(void* h, int* out, int cap) {
  auto* s = static_cast<Scheduler*>(h);
  const int n = std::min<int>(cap, static_cast<int>(s->recorded.size()));
  for (int i = 0; i < n; ++i) {
    out[4 * i] = s->recorded[i].kind; out[4 * i + 1] = s->recorded[i].layer;
    out[4 * i + 2] = s->recorded[i].expert; out[4 * i + 3] = s->recorded[i].gpu;
  }
  s->recorded.erase(s->recorded.begin(), s->recorded.begin() + n);
  return n;
}

// ---- accuracy tracker ------------------------------------------------------------------------------------------------
void* ihb_acc_create(int n_layers, int top_k) {
  return new Accuracy{n_layers, top_k, std::vector<uint64_t>(n_layers, 0), std::vector<uint64_t>(n_layers, 0)};
}
void ihb_acc_destroy(void* h) { delete static_cast<Accuracy*>(h); }
void ihb_acc_record(void* h, int layer, const int* predicted, int n_pred, const int* actual, int n_actual) {
  auto* a = static_cast<Accuracy*>(h);
  if (layer < 0 || layer >= a->n_layers) return;
  for (int i = 0; i < n_pred; ++i)
    if (std::find(actual, actual + n_actual, predicted[i]) != actual + n_actual) ++a->hits[layer];
  a->total[layer] += a->top_k;
}
float ihb_acc_hit_rate(void* h, int layer) {
  auto* a = static_cast<Accuracy*>(h);
  if (layer < 0 || layer >= a->n_layers) return 0.f;
  return a->total[layer] ? static_cast<float>(a->hits[layer]) / static_cast<float>(a->total[layer]) : 0.f;
}
unsigned long long ihb_acc_tokens(void* h, int layer) {
  auto* a = static_cast<Accuracy*>(h);
  if (layer < 0 || layer >= a->n_layers) return 0;
  return a->top_k ? a->total[layer] / a->top_k : 0;
}
float ihb_acc_mean_hit_rate(void* h) {
  auto* a = static_cast<Accuracy*>(h);
  float sum = 0.f;
  int n = 0;
  for (int l = 0; l < a->n_layers; ++l)
    if (a->total[l]) { sum += ihb_acc_hit_rate(h, l); ++n; }
  return n ? sum / n : 0.f;
}
void ihb_acc_reset(void* h) {
  auto* a = static_cast<Accuracy*>(h);
  std::fill(a->hits.begin(), a->hits.end(), 0);
  std::fill(a->total.begin(), a->total.end(), 0);
}

// ---- trace collector ---------------------------------------------------------------------------------------------------
void* ihb_trace_create(int hidden, int n_experts, int max_traces) { return new Traces{hidden, n_experts, max_traces, {}, {}, {}}; }
void ihb_trace_destroy(void* h) { delete static_cast<Traces*>(h); }
int ihb_trace_push(void* h, int layer, const float* hidden, const float* logits) {
  auto* t = static_cast<Traces*>(h);
  if (static_cast<int>(t->layers.size()) >= t->max_traces) return 0;
  t->h.insert(t->h.end(), hidden, hidden + t->hidden);
  t->logits.insert(t->logits.end(), logits, logits + t->n_experts);
  t->layers.push_back(layer);
  return 1;
}
int ihb_trace_count(void* h, int layer) {
  auto* t = static_cast<Traces*>(h);
  if (layer < 0) return static_cast<int>(t->layers.size());
  return static_cast<int>(std::count(t->layers.begin(), t->layers.end(), layer));
}
// copies the traces of `layer` into the outputs (sized by ihb_trace_count) and removes them, keeping the rest in order
int ihb_trace_drain_layer(void* h, int layer, float* out_hidden, float* out_logits) {
  auto* t = static_cast<Traces*>(h);
  int n = 0;
  size_t keep = 0;
  for (size_t i = 0; i < t->layers.size(); ++i) {
    const float* hs = &t->h[i * t->hidden];
    const float* lg = &t->logits[i * t->n_experts];
    if (t->layers[i] == layer) {
      std::memcpy(out_hidden + static_cast<size_t>(n) * t->hidden, hs, sizeof(float) * t->hidden);
      std::memcpy(out_logits + static_cast<size_t>(n) * t->n_experts, lg, sizeof(float) * t->n_experts);
      ++n;
    } else {
      if (keep != i) {
        std::memmove(&t->h[keep * t->hidden], hs, sizeof(float) * t->hidden);
        std::memmove(&t->logits[keep * t->n_experts], lg, sizeof(float) * t->n_experts);
        t->layers[keep] = t->layers[i];
      }
      ++keep;
    }
  }
  t->layers.resize(keep);
  t->h.resize(keep * t->hidden);
  t->logits.resize(keep * t->n_experts);
  return n;
}
void ihb_trace_clear(void* h) {
  auto* t = static_cast<Traces*>(h);
  t->h.clear(); t->logits.clear(); t->layers.clear();
}

}  // extern "C"
