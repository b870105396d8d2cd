// Argument block shared by the forward kernels and the host launcher.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <vector_types.h>

namespace ma {

struct FwdArgs {
  float*   lse;        // [B, Hq, Nq] or null
  int32_t* status;     // device word for wait-timeout bits, or null
  long long q_pos0;    // global position of query token 0
  long long k_pos0;    // global position of key token 0
  int Nq, Nk, Hq, Hkv, B;
  int causal;
  float scale;         // softmax scale
  float scale_log2;    // softmax scale * log2(e)
  int n_q_tiles;       // ceil(Nq / 128)
  int n_pair_items;    // warp-specialised kernel: CTAs [0, n_pair_items) take two Q tiles each,
                       // the CTAs after them one Q tile each (the tail of the last wave)
  int bh_group;        // work items are ordered in groups of this many consecutive (batch, head)
                       // indices: all Q-tile pairs of a group (latest first, heads fastest) before the
                       // next group.  B*Hq = one group, the default order.  Divides B*Hq.
  const float* sq;     // INT8-QK: [B, Hq,  ceil(Nq/128)] Q scales (softmax scale * log2e folded in)
  const float* sk;     // INT8-QK: [B, Hkv, ceil(Nk/128)] K scales
  // Balanced launches only (null otherwise): where CTAs that cover part of an item's key range
  // leave their partial result, and the per-item arrival counters (zero between launches).
  float*  part_o;      // [slot][2 tiles][D/4][128 rows][4] fp32, un-normalised O of a piece
  float2* part_ml;     // [slot][2 tiles][128 rows]: (row maximum in log2 units, row sum)
  int*    counters;    // [cut item][2 tiles][arrived, published]
  // Ring steps only (carry_mode != 0): the rows' running state between launches.
  float*  carry_o;     // [B*Hq*carry_tiles][D/4][128 rows][4] fp32, un-normalised O
  float2* carry_ml;    // [B*Hq*carry_tiles][128 rows]: (row maximum in log2 units, row sum)
  int     carry_mode;  // bit 0: fold the stored state in; bit 1: store the new state, no output
  int     carry_tile0; // the state holds carry_tiles tiles per (batch, head); this launch's first
  int     carry_tiles; // Q tile is number carry_tile0 of them
};

// One CTA of a balanced launch, read from the launch's table (kernel parameter space).
struct PlanEntry {
  uint32_t item;         // index in the heaviest-first item order
  uint16_t t0, t1;       // the CTA covers K/V tiles [t0, t1) of the item
  uint16_t slot0;        // first partial slot of the item (its pieces hold consecutive slots)
  uint8_t  part, nparts; // nparts == 1: whole item, the CTA writes the output itself
  uint32_t counter;      // arrival-counter index of a cut item
};
constexpr int kPlanCap = 768;
struct PlanTable { PlanEntry e[kPlanCap]; };
struct NoPlanTable { int unused; };

// Result of the host-side planner (plan.cu).
struct FwdPlan {
  bool split;            // false: launch the items as they are
  int n_whole;           // CTAs [0, n_whole) take items [0, n_whole) whole
  int n_table;           // the CTAs after them read table.e[cta - n_whole]
  int n_slots;           // partial slots the launch writes
  int n_cut_items;       // items covered by more than one CTA
  float est_plain;       // predicted makespans, in K/V-tile steps of one CTA
  float est_balanced;
  PlanTable table;
};

constexpr int kTileM = 128;   // query rows per MMA tile (TMEM lanes)
constexpr int kTileN = 128;   // keys per K/V tile
constexpr int kBoxCols = 64;  // 16-bit elements per 128-byte swizzled row
constexpr int kBoxBytes = kTileN * 128;  // one [128 rows x 128 B] TMA box

// Work item -> (Q-tile pair, (batch, head) index).  Items walk the (batch, head) indices in groups
// of a.bh_group: within a group the latest Q-tile pair first (the heaviest under a causal mask) and
// heads fastest, so that the CTAs in flight share the K/V of few heads.  Shared by the kernels and
// the host planner.
__host__ __device__ inline void item_to_pair_bh(const FwdArgs& a, int n_pairs, int item, int* pair, int* bh) {
  const int per_group = n_pairs * a.bh_group;
  const int within = item % per_group;
  *pair = n_pairs - 1 - within / a.bh_group;
  *bh = (item / per_group) * a.bh_group + within % a.bh_group;
}

// Number of K/V tiles the Q rows [q0, q0 + nt*128) have to visit (all of them without a mask,
// up to the diagonal of the last row with one).  Shared by the kernels and the host planner.
__host__ __device__ inline int kv_tiles_of(const FwdArgs& a, int q0, int nt) {
  long long kv_end = a.Nk;
  if (a.causal) {
    long long last_row = q0 + nt * kTileM - 1;
    if (last_row > a.Nq - 1) last_row = a.Nq - 1;
    long long vis = a.q_pos0 + last_row - a.k_pos0 + 1;
    if (vis < kv_end) kv_end = vis;
    if (kv_end < 0) kv_end = 0;
  }
  return static_cast<int>((kv_end + kTileN - 1) / kTileN);
}

}  // namespace ma
