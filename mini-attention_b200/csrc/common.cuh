// Argument block shared by the forward kernels and the host launcher.
#pragma once
#include <cstdint>
#include <cuda.h>

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
  const float* sq;     // INT8-QK: [B, Hq,  ceil(Nq/128)] Q scales (softmax scale * log2e folded in)
  const float* sk;     // INT8-QK: [B, Hkv, ceil(Nk/128)] K scales
  unsigned long long* trace;  // debug builds only (MA_TRACE): per-role clock stamps of CTA 0
};

constexpr int kTileM = 128;   // query rows per MMA tile (TMEM lanes)
constexpr int kTileN = 128;   // keys per K/V tile
constexpr int kBoxCols = 64;  // 16-bit elements per 128-byte swizzled row
constexpr int kBoxBytes = kTileN * 128;  // one [128 rows x 128 B] TMA box

}  // namespace ma
