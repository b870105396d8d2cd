// Host-side planner of balanced launches.
//
// The forward kernel runs one CTA per SM, so a launch of n work items (pairs of Q tiles of one
// (batch, head)) takes ceil(n / SMs) rounds when the items are equally heavy, and the last round
// may leave most SMs idle (256 items on 148 SMs: 2 rounds for 1.73 rounds of work).  The planner
// cuts the K/V range of some items into pieces that separate CTAs work on, so that every SM ends
// at about the same time; the CTAs of a cut item leave un-normalised partial results in scratch
// memory and the last one to arrive merges them (fwd_ws.cu).  The reference launches one CTA per
// (batch, head, Q block) and leaves the balance to the hardware scheduler
// (kernels/flash_attn/cuda/sm_120/kernel/flash_attention.cu:100-123).
//
// Model: a CTA covering s K/V tiles costs s + h steps (h = fixed cost of a CTA: set-up, first
// loads, epilogue); the hardware hands CTAs to SMs in index order as SMs become free.  Plan:
// walk the items heaviest first and give each to the least-loaded SM while it fits under the
// target time T; from the first item that does not fit, fill the SMs one after the other up to T,
// cutting an item where an SM's room ends and continuing it on the next SM (McNaughton's
// wrap-around rule, with a minimum piece length).  The resulting CTAs are launched
// longest first.  The plan is used only when its predicted makespan beats the plain launch.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <functional>
#include <queue>
#include <utility>
#include <vector>

#include "common.cuh"

namespace ma {

namespace {

struct Piece {
  int item, t0, t1, part, nparts;
  int round;  // how many pieces the plan put on the same SM before this one (phase 2)
};

using SmLoad = std::pair<float, int>;  // (busy until, SM)
using MinHeap = std::priority_queue<SmLoad, std::vector<SmLoad>, std::greater<SmLoad>>;

MinHeap empty_sms(int sms) {
  std::vector<SmLoad> v;
  v.reserve(sms);
  for (int s = 0; s < sms; ++s) v.emplace_back(0.f, s);
  return MinHeap(std::greater<SmLoad>(), std::move(v));
}

// Makespan of CTAs with the given costs, handed out in order to the first free SM; `finish`
// (optional) receives the time each CTA ends.
float list_schedule(const std::vector<float>& cost, int sms, std::vector<float>* finish = nullptr) {
  MinHeap heap = empty_sms(sms);
  float end = 0.f;
  if (finish) finish->resize(cost.size());
  for (size_t i = 0; i < cost.size(); ++i) {
    SmLoad s = heap.top();
    heap.pop();
    s.first += cost[i];
    if (finish) (*finish)[i] = s.first;
    end = std::max(end, s.first);
    heap.push(s);
  }
  return end;
}

constexpr int kMinPiece = 6;       // K/V tiles; shorter pieces cost more than they balance (measured: a 4-tile piece loses)
constexpr int kMaxParts = 64;      // pieces per item

// Cost model, in steps (one K/V tile of a two-Q-tile CTA, about 2 us at D = 128): fixed cost of
// a CTA, and what a piece of a cut item adds on average (publishing its partial takes about 0.6
// steps; the last piece to arrive also reads the others', about 2 steps).
float cta_cost(int D) { return D == 128 ? 2.0f : 3.0f; }
float grade_frac() { return 0.015f; }  // spread of the per-SM targets, as a fraction of T
float piece_cost() { return 1.3f; }

// Fill under the target time T.  Phase 1: items go whole to the least-loaded SM while they fit.
// Phase 2, from the first item that does not: the SMs are filled one after the other up to T
// (most room first); an item that crosses the end of an SM's room is cut there and continues on
// the next SM.  Returns false when an item would need too many pieces.
bool fill(const std::vector<int>& w, int sms, float T, float h, float fee, std::vector<Piece>* out) {
  out->clear();
  const int n = static_cast<int>(w.size());
  MinHeap heap = empty_sms(sms);
  int i = 0;
  for (; i < n; ++i) {
    SmLoad s = heap.top();
    if (s.first + w[i] + h > T) break;
    heap.pop();
    out->push_back(Piece{i, 0, w[i], 0, 1, 0});
    s.first += w[i] + h;
    heap.push(s);
  }
  std::vector<float> load;
  load.reserve(sms);
  while (!heap.empty()) {
    load.push_back(heap.top().first);  // ascending: most room first
    heap.pop();
  }
  std::vector<int> placed(sms, 0);
  const float grade = grade_frac() * T;
  int si = 0;
  for (; i < n; ++i) {
    int t0 = 0;
    const size_t first = out->size();
    do {
      const int rem = w[i] - t0;
      int take, round;
      if (si >= sms) {
        // no SM has room left under T: the rest goes, in one piece, to the least-loaded SM
        const int s = static_cast<int>(std::min_element(load.begin(), load.end()) - load.begin());
        take = rem;
        load[s] += take + h + (t0 > 0 ? fee : 0.f);
        round = placed[s]++;
      } else {
        take = rem;
        // SMs do not run identical CTAs at identical speed (a few per cent apart), and CTAs are
        // handed out longest first to whichever SM is free first.  Grading the targets, more for
        // the SMs filled first, gives the SMs that come free early the longer pieces.
        const float Ts = T + grade * (1.f - 2.f * si / std::max(1, sms - 1));
        const bool whole_fits = (t0 == 0) && (load[si] + rem + h <= Ts);
        if (!whole_fits) {  // a piece of a cut item: it also pays the fee
          const int room = static_cast<int>(std::floor(Ts - load[si] - h - fee));
          if (room < rem) {
            if (room < kMinPiece) {
              ++si;  // nothing useful fits here any more
              continue;
            }
            // both sides of a cut at least kMinPiece long; a rest too short to cut stays whole
            // (and overruns this SM's target by less than kMinPiece)
            if (rem >= 2 * kMinPiece) take = std::min(room, rem - kMinPiece);
          }
        }
        load[si] += take + h + (whole_fits ? 0.f : fee);
        round = placed[si]++;
        if (Ts - load[si] - h - fee < kMinPiece) ++si;
      }
      out->push_back(Piece{i, t0, t0 + take, 0, 0, round});
      t0 += take;
    } while (t0 < w[i]);
    const int np = static_cast<int>(out->size() - first);
    if (np > kMaxParts) return false;
    for (int k = 0; k < np; ++k) {
      (*out)[first + k].part = k;
      (*out)[first + k].nparts = np;
    }
  }
  return true;
}

}  // namespace

// Items in launch order (item_to_pair_bh): latest rows first within each group of heads.
void plan_fwd(const FwdArgs& a, int D, int sms, FwdPlan* plan) {
  plan->split = false;
  plan->n_whole = plan->n_table = plan->n_slots = plan->n_cut_items = 0;
  plan->est_plain = plan->est_balanced = 0.f;
  const long long n_pairs = (a.n_q_tiles + 1) / 2;
  const long long bh = static_cast<long long>(a.Hq) * a.B;
  const long long n_items = n_pairs * bh;
  // Many rounds balance themselves; the table holds every CTA from the first cut item on.
  if (sms <= 0 || n_items <= 0 || n_items > 16ll * sms || n_items > 4096) return;
  const int n = static_cast<int>(n_items);
  const float h = cta_cost(D);
  const float fee = piece_cost();

  std::vector<int> w(n);
  long long total = 0;
  for (int i = 0; i < n; ++i) {
    int pair, bh_i;
    item_to_pair_bh(a, static_cast<int>(n_pairs), i, &pair, &bh_i);
    const int q0 = pair * 2 * kTileM;
    const int nt = (q0 + kTileM < a.Nq) ? 2 : 1;
    w[i] = kv_tiles_of(a, q0, nt);
    if (w[i] > 65535) return;  // tile ranges travel as 16-bit numbers
    total += w[i];
  }
  std::vector<float> cost(n);
  for (int i = 0; i < n; ++i) cost[i] = w[i] + h;
  const float plain = list_schedule(cost, sms);
  plan->est_plain = plain;
  const float bound = (static_cast<float>(total) + h * n) / sms;
  if (plain <= 1.03f * bound) return;

  std::vector<Piece> best, cur;
  float best_t = plain;
  int best_whole = 0;
  // Targets tried: ten fine steps above the bound (several rounds of items: the answer is close
  // to it), then eight coarse ones up to about half the heaviest item (few, long items).
  const int w_max = *std::max_element(w.begin(), w.end());
  const float fine = std::max(0.5f, 0.004f * bound), coarse = std::max(fine, w_max / 16.f);
  for (int attempt = 0; attempt < 18; ++attempt) {
    const float up = attempt < 10 ? fine * attempt : fine * 9 + coarse * (attempt - 9);
    const float T = std::max(bound + 0.75f * (h + fee) + up, kMinPiece + h + fee);
    if (!fill(w, sms, T, h, fee, &cur)) continue;
    int first_cut = n;
    for (const Piece& p : cur)
      if (p.nparts > 1) {
        first_cut = p.item;
        break;
      }
    if (first_cut == n) continue;  // nothing was cut
    // Launch order: the whole items before the first cut one, then everything else, either
    // longest first, or in the plan's rounds (first pieces of every SM, longest first, then the
    // second pieces, ...); whichever the dispatch model likes better.
    std::vector<Piece> tab;
    for (const Piece& p : cur)
      if (p.item >= first_cut) tab.push_back(p);
    if (static_cast<int>(tab.size()) > kPlanCap) continue;
    for (int order = 0; order < 2; ++order) {
      std::stable_sort(tab.begin(), tab.end(), [order](const Piece& x, const Piece& y) {
        if (order == 1 && x.round != y.round) return x.round < y.round;
        return (x.t1 - x.t0) > (y.t1 - y.t0);
      });
      // Every piece of a cut item publishes its partial; the one that ends last also merges.
      // Two passes: who ends last is read off a first schedule in which nobody pays the merge.
      const float fee_pub = 0.45f * fee, fee_last = 1.55f * fee;
      std::vector<float> c, fin;
      c.reserve(first_cut + tab.size());
      for (int i = 0; i < first_cut; ++i) c.push_back(w[i] + h);
      for (const Piece& p : tab) c.push_back((p.t1 - p.t0) + h + (p.nparts > 1 ? fee_pub : 0.f));
      list_schedule(c, sms, &fin);
      std::vector<int> last_of(n, -1);
      for (size_t k = 0; k < tab.size(); ++k) {
        const Piece& p = tab[k];
        if (p.nparts > 1 && (last_of[p.item] < 0 || fin[first_cut + k] > fin[first_cut + last_of[p.item]]))
          last_of[p.item] = static_cast<int>(k);
      }
      for (size_t k = 0; k < tab.size(); ++k)
        if (tab[k].nparts > 1 && last_of[tab[k].item] == static_cast<int>(k)) c[first_cut + k] += fee_last - fee_pub;
      const float t = list_schedule(c, sms);
      if (t < best_t) {
        best_t = t;
        best_whole = first_cut;
        best = tab;
      }
    }
  }
  plan->est_balanced = best_t;
  if (best.empty() || best_t > 0.97f * plain) return;

  // slots and counters: cut items in item order, pieces of an item on consecutive slots
  std::vector<int> slot0(n, -1), counter(n, -1);
  {
    std::vector<int> nparts(n, 0);
    for (const Piece& p : best) nparts[p.item] = p.nparts;
    int slots = 0, cuts = 0;
    for (int i = best_whole; i < n; ++i)
      if (nparts[i] > 1) {
        slot0[i] = slots;
        counter[i] = cuts++;
        slots += nparts[i];
      }
    if (slots > 65535) return;
    plan->n_slots = slots;
    plan->n_cut_items = cuts;
  }
  plan->split = true;
  plan->n_whole = best_whole;
  plan->n_table = static_cast<int>(best.size());
  for (int k = 0; k < plan->n_table; ++k) {
    const Piece& p = best[k];
    PlanEntry& e = plan->table.e[k];
    e.item = static_cast<uint32_t>(p.item);
    e.t0 = static_cast<uint16_t>(p.t0);
    e.t1 = static_cast<uint16_t>(p.t1);
    e.part = static_cast<uint8_t>(p.part);
    e.nparts = static_cast<uint8_t>(p.nparts);
    e.slot0 = static_cast<uint16_t>(p.nparts > 1 ? slot0[p.item] : 0);
    e.counter = static_cast<uint32_t>(p.nparts > 1 ? counter[p.item] : 0);
  }
}

}  // namespace ma
