// Forward attention, warp-specialised sm_100a kernel.
//
// One CTA (512 threads) per work item = two 128-row Q tiles of one (batch, head).  Same math as
// the reference mainloop (kernels/flash_attn/cuda/sm_120/kernel/include/forward_kernel.cuh:137-221
// and softmax.cuh:29-138), restructured for tcgen05 / TMEM / TMA:
//
//   warps 0-3   softmax of Q tile 0   (thread = one query row; S row read from TMEM), then its
//               epilogue (O / l -> 16 bit -> swizzled smem -> TMA store)
//   warps 4-7   softmax and epilogue of Q tile 1
//   warps 8-11  correction: rescales the O accumulators in TMEM when a row maximum moved (rare)
//   warp 12     MMA issuer of Q tile 0 (one thread issues its tcgen05.mma stream)
//   warp 14     MMA issuer of Q tile 1
//   warp 13     TMA producer: Q tiles once, then K_0, V_0, K_1, V_1, ... through a ring
//   warp 15     idle (donates its registers)
//
// A 128-key K/V tile is worked on as two 64-key halves ("a", "b").  Each Q tile owns two S
// buffers of 64 TMEM columns; the 16-bit P of a half overwrites the first 32 columns of its own
// S buffer and feeds the PV MMA straight from TMEM (A operand).  Because the halves have separate
// buffers, S_half(j+1) is computed while the softmax group still works on the other half, so the
// softmax never waits for the chain  P -> PV -> next S  of the half it just finished.
//
// TMEM (512 columns x 128 lanes x 32 bit):
//   S0a [0,64) S0b [64,128) S1a [128,192) S1b [192,256)   O0 [256,256+D)  O1 [256+D,256+2D)
//
// MMA order per Q tile and K/V tile j:  PV_a(j) S_a(j+1) PV_b(j) S_b(j+1); the two tiles have
// one issuing thread each and the tensor pipe interleaves their streams.
//
// The row maximum is updated lazily: a row keeps exponentiating against a stale maximum until the
// true maximum has grown by more than 2^8 (in the exp2 domain), so the O accumulator is rescaled
// only rarely; l is accumulated against the same maximum, which keeps O / l exact.
//
// Softmax arithmetic runs two scores per issue slot (packed f32x2 FMA / ADD); a share of the
// exponentials is evaluated by a cubic on the FMA pipe instead of the exp2 unit.
//
// Template variants of the one kernel: QK8 (int8 Q K^T, accumulator pre-biased so that the scores
// arrive as floats), PLAN (balanced launch: work items cut over several CTAs, merged by the last
// to arrive), CARRY (ring steps: the rows' running state is read from and written to global
// memory in the epilogue instead of a second, merging launch).
#include <atomic>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace ma {

namespace {

constexpr int kNumThreads = 512;
constexpr int kHalfN = kTileN / 2;      // keys per half tile
constexpr float kLazyThreshold = 8.0f;  // log2 units
// Register split per thread after setmaxnreg (8 softmax + 4 correction + 4 other warps;
// 8*176 + 4*88 + 4*72 = 2048 = the 64 K registers of an SM divided by 32 lanes).
constexpr int kRegSoftmax = 176;
constexpr int kRegCorr = 88;
constexpr int kRegOther = 72;

template <int D, bool QK8 = false>
struct WsLayout {
  static constexpr int kBoxes = D / kBoxCols;
  static constexpr int kTileBytes = kBoxes * kBoxBytes;  // Q, K or V tile (32 KB at D=128)
  static constexpr int kStages = (D == 128) ? 4 : 8;     // ring slots, each one K or V tile
  static constexpr int kOffQ = 0;                        // two Q tiles (reused as O staging)
  static constexpr int kOffRing = 2 * kTileBytes;
  // INT8-QK only: two constant fp16 operand tiles (A: 128 rows, B: 64 rows, 128-byte swizzled
  // rows) whose product is 1.5 * 2^23 in every element, see issue_s
  static constexpr int kOffBiasA = kOffRing + kStages * kTileBytes;
  static constexpr int kOffBiasB = kOffBiasA + kTileM * 128;
  static constexpr int kBiasBytes = QK8 ? (kTileM + kTileN / 2) * 128 : 0;
  static constexpr int kOffAlpha = kOffBiasA + kBiasBytes;           // float[2 tiles][2 halves][128]
  static constexpr int kOffL = kOffAlpha + 2048;                     // float[2][128]
  static constexpr int kOffBar = kOffL + 1024;
  // barrier indices (8 bytes each); [t][h] = index + 2*t + h
  static constexpr int kBarQFull = 0;                      // [2]
  static constexpr int kBarKvFull = 2;                     // [kStages]
  static constexpr int kBarKvEmpty = kBarKvFull + kStages; // [kStages]
  static constexpr int kBarSFull = kBarKvEmpty + kStages;  // [2][2] MMA -> softmax
  static constexpr int kBarPReady = kBarSFull + 4;         // [2][2] softmax -> MMA
  static constexpr int kBarAlpha = kBarPReady + 4;         // [2][2] softmax -> correction
  static constexpr int kBarOReady = kBarAlpha + 4;         // [2][2] correction -> MMA
  static constexpr int kBarODone = kBarOReady + 4;         // [2][2] MMA -> correction
  static constexpr int kBarStagger = kBarODone + 4;        // one-shot: tile 0 published its first row maxima
  static constexpr int kNumBars = kBarStagger + 1;
  static constexpr int kOffMisc = kOffBar + kNumBars * 8;  // tmem slot, abort flag, arrival order [2]
  static constexpr int kBytes = kOffMisc + 32;
  static constexpr int kDynSmem = kBytes + 1024;
  static constexpr int kTmemCols = 512;
  static constexpr int kColS = 0;     // S buffer of (tile t, half h) at kColS + 128*t + 64*h
  static constexpr int kColO = 256;   // O accumulator of tile t at kColO + D*t
};

constexpr int kBarEpilogue = 1;  // named barriers 1 and 2: epilogue of softmax group 0 / 1
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
template <int N>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
__device__ __forceinline__ void warp_arrive(uint32_t bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}

}  // namespace

// QK8: Q and K arrive as int8 (one fp32 scale per 128-token block, softmax scale * log2e folded
// into the Q scales); S = Q8 K8^T runs on tcgen05 kind::i8 with an int32 accumulator and is
// de-quantised on the fly in the softmax; P, V and the PV MMA stay 16 bit.
//
// PLAN: balanced launch.  CTAs past the first a.n_pair_items read their work from `plan`: an item
// and a range of its K/V tiles.  The CTAs that share an item each leave their un-normalised O and
// (row maximum, row sum) in scratch memory, count themselves in on the item's arrival counter, and
// the one that arrives last folds the others' partials into its own and writes the output; nobody
// waits for another CTA.
//
// CARRY: ring (context-parallel) steps.  The rows' running state over the key blocks seen so far
// -- un-normalised O (fp32, the layout of a balanced launch's partial) and (row maximum, row sum)
// -- lives in global memory between launches.  With a.carry_mode bit 0 the epilogue folds that state
// into this launch's result; with bit 1 it writes the new state instead of the 16-bit output.
template <int D, bool BF16, bool QK8, bool PLAN, bool CARRY = false>
__global__ void __launch_bounds__(kNumThreads, 1)
fwd_ws_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
              const FwdArgs a,
              const __grid_constant__ std::conditional_t<PLAN, PlanTable, NoPlanTable> plan) {
  using L = WsLayout<D, QK8>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (sbase - raw);

  const uint32_t sQ = sbase + L::kOffQ;
  const uint32_t sRing = sbase + L::kOffRing;
  float* alpha_smem = reinterpret_cast<float*>(gbase + L::kOffAlpha);
  const uint32_t bars = sbase + L::kOffBar;
  auto bar = [&](int idx) -> uint32_t { return bars + 8u * idx; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + L::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + L::kOffMisc + 8);
  volatile int* arrival = reinterpret_cast<volatile int*>(gbase + L::kOffMisc + 16);  // [2 tiles]

  const int tid = threadIdx.x;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // warp-uniform for the compiler
  const int lane = tid & 31;

  // ---- work item: heaviest (latest) Q tile pairs first; heads of one pair adjacent ----
  // CTAs past n_pair_items take a single Q tile: the launcher cuts the pairs that would form a
  // less-than-half-full last wave into two CTAs each, so that the wave ends sooner.
  const int n_pairs = (a.n_q_tiles + 1) >> 1;
  const int bh_total = a.Hq * a.B;
  int item = blockIdx.x;
  int single = -1;  // which tile of its pair a single-tile CTA takes
  int pe_t0 = 0, pe_t1 = -1, pe_part = 0, pe_nparts = 1, pe_slot0 = 0, pe_counter = 0;
  if (item >= a.n_pair_items) {
    if constexpr (PLAN) {
      const PlanEntry& e = plan.e[item - a.n_pair_items];
      item = static_cast<int>(e.item);
      pe_t0 = e.t0;
      pe_t1 = e.t1;
      pe_part = e.part;
      pe_nparts = e.nparts;
      pe_slot0 = e.slot0;
      pe_counter = static_cast<int>(e.counter);
    } else {
      const int s_idx = item - a.n_pair_items;
      item = a.n_pair_items + (s_idx >> 1);
      single = s_idx & 1;
    }
  }
  int pair, bh;
  item_to_pair_bh(a, n_pairs, item, &pair, &bh);
  const int h = bh % a.Hq;
  const int b = bh / a.Hq;
  const int hk = h / (a.Hq / a.Hkv);
  const int q0 = (pair * 2 + (single > 0 ? 1 : 0)) * kTileM;
  // Q tiles of this CTA that hold real rows
  const int nt = (single < 0 && q0 + kTileM < a.Nq) ? 2 : 1;

  // K/V tiles [kv_t0, kv_t0 + n_tiles) of this CTA: all the rows can see, or the table's range
  int kv_end = a.Nk;
  if (a.causal) {
    const int last_row = min(q0 + nt * kTileM - 1, a.Nq - 1);
    const long long vis = a.q_pos0 + last_row - a.k_pos0 + 1;
    kv_end = static_cast<int>(max(0ll, min(static_cast<long long>(a.Nk), vis)));
  }
  int kv_t0 = 0;
  int n_tiles = (kv_end + kTileN - 1) / kTileN;  // == kv_tiles_of(a, q0, nt)
  if (PLAN && pe_t1 >= 0) {
    kv_t0 = pe_t0;
    n_tiles = pe_t1 - pe_t0;
  }

  // TMA loads (issued by lane 0 of warp 13 only): Q tile t; ring fill i = K (even) or V (odd) of
  // K/V tile kv_t0 + i/2 into slot i % kStages.
  auto load_q = [&](int t) {
    if constexpr (QK8) {  // one box of D bytes x 128 rows
      mbar_expect_tx(bar(L::kBarQFull + t), kTileM * D);
      tma_load_4d(sQ + t * L::kTileBytes, &tm_q, bar(L::kBarQFull + t), 0, q0 + t * kTileM, h, b);
    } else {
      mbar_expect_tx(bar(L::kBarQFull + t), L::kTileBytes);
#pragma unroll
      for (int bx = 0; bx < L::kBoxes; ++bx)
        tma_load_4d(sQ + t * L::kTileBytes + bx * kBoxBytes, &tm_q, bar(L::kBarQFull + t),
                    bx * kBoxCols, q0 + t * kTileM, h, b);
    }
  };
  auto load_kv = [&](int i) {
    const int slot = i % L::kStages;
    const uint32_t fb = bar(L::kBarKvFull + slot);
    const int j = kv_t0 + (i >> 1);
    if (QK8 && !(i & 1)) {  // int8 K tile: one box of D bytes x 128 rows
      mbar_expect_tx(fb, kTileN * D);
      tma_load_4d(sRing + slot * L::kTileBytes, &tm_k, fb, 0, j * kTileN, hk, b);
    } else {
      mbar_expect_tx(fb, L::kTileBytes);
      const CUtensorMap* tm = (i & 1) ? &tm_v : &tm_k;
#pragma unroll
      for (int bx = 0; bx < L::kBoxes; ++bx)
        tma_load_4d(sRing + slot * L::kTileBytes + bx * kBoxBytes, tm, fb, bx * kBoxCols, j * kTileN, hk, b);
    }
  };
  const int n_fill = 2 * n_tiles;
  const int n_early = min(n_fill, L::kStages);  // first use of every ring slot: nothing to wait for

  if (warp == 13) {
    // one barrier per lane: arrival counts by index range
    for (int i = lane; i < L::kNumBars; i += 32) {
      uint32_t count = 1;  // Q full, K/V full, S full, O done: one arrival (a TMA or MMA commit)
      if (i >= L::kBarKvEmpty && i < L::kBarSFull) count = nt;      // one release per issuing thread
      else if (i >= L::kBarPReady && i < L::kBarODone) count = 4;   // P ready, alpha, O ready: 4 warps
      else if (i == L::kBarStagger) count = 4;                      // the 4 softmax warps of tile 0, once
      mbar_init(bar(i), count);
    }
    if (lane == 0) *abort_flag = 0;
    fence_mbar_init();
    __syncwarp();
  }
  if (warp == 13 && lane == 0) {
    fence_proxy_async_smem();
    // The first loads start here, before TMEM is allocated and the CTA synchronises: their
    // latency overlaps the rest of the set-up.
    if (n_tiles > 0) {
      for (int t = 0; t < nt; ++t) load_q(t);
      for (int i = 0; i < n_early; ++i) load_kv(i);
    }
    prefetch_tmap(&tm_o);
  }
  if (warp == 12) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), L::kTmemCols);
    tmem_relinquish();
  }
  if constexpr (QK8) {
    // Bias operands: row r of a 128-byte swizzled tile keeps its logical 16-byte chunk 0 at
    // physical chunk (r & 7); element k = 0 of every row is 3072 (A) or 4096 (B), the rest 0.
    uint4* bias = reinterpret_cast<uint4*>(gbase + L::kOffBiasA);
    for (int i = tid; i < L::kBiasBytes / 16; i += kNumThreads) {
      const int r = i >> 3, chunk = i & 7;
      const uint32_t v = (r < kTileM) ? 0x6A00u : 0x6C00u;  // fp16 3072.0 / 4096.0
      bias[i] = make_uint4(chunk == (r & 7) ? v : 0u, 0u, 0u, 0u);
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const WaitCtx wc{abort_flag, a.status, MINIATTN_WAIT_LIMIT_NS};
  const float c = a.scale_log2;

  if (warp < 8) {
    // =========================== softmax ===========================================
    reg_inc<kRegSoftmax>();
    const int t = warp >> 2;
    if (t < nt) {
      const int r = tid & 127;
      const int row = q0 + t * kTileM + r;
      const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const uint32_t tS = tmem_base + L::kColS + 128 * t + lane_off;
      long long vis_ll = a.Nk;
      if (a.causal) vis_ll = min(vis_ll, a.q_pos0 + row - a.k_pos0 + 1);
      const int vis_row = static_cast<int>(max(0ll, vis_ll));
      float m_cur = -INFINITY;  // running (lazily updated) row maximum, log2 units
      float l_run = 0.f;
      float sq_t = 0.f, sk_next = 0.f;
      const float* sk_row = nullptr;
      if constexpr (QK8) {
        sq_t = __ldg(a.sq + (static_cast<long long>(b) * a.Hq + h) * a.n_q_tiles + (q0 / kTileM + t));
        sk_row = a.sk + (static_cast<long long>(b) * a.Hkv + hk) * ((a.Nk + kTileN - 1) / kTileN);
        sk_row += kv_t0;
        if (n_tiles > 0) sk_next = __ldg(sk_row);
      }

      for (int j = 0; j < n_tiles; ++j) {
        // cj turns a raw score into log2 units: softmax scale * log2e, times the two
        // de-quantisation scales of this (Q block, K block) for the int8 variant.
        float cj = c;
        if constexpr (QK8) {
          cj = sq_t * sk_next;
          if (j + 1 < n_tiles) sk_next = __ldg(sk_row + j + 1);
        }
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
          mbar_wait(bar(L::kBarSFull + 2 * t + hb), j & 1, wc, kErrWaitS);
          tc_fence_after();
          uint32_t s[2][32];
          tmem_ld32(tS + hb * kHalfN, s[0]);
          tmem_ld32(tS + hb * kHalfN + 32, s[1]);
          tmem_wait_ld();
          // QK8: the accumulator was started at the bit pattern of 1.5*2^23 (see issue_s) and
          // |acc| <= 127*127*D < 2^22, so the word read here IS the float 12582912 + acc: int32 ->
          // fp32 with no instruction at all.  The offset stays in: it is order-preserving for the
          // maximum and folds into the constant of the exp2 FMA.
          const int lim = vis_row - (kv_t0 + j) * kTileN - hb * kHalfN;
          if (lim < kHalfN) {  // diagonal or ragged half: hide the keys this row must not see
#pragma unroll
            for (int q = 0; q < 2; ++q)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (q * 32 + i >= lim) s[q][i] = __float_as_uint(-INFINITY);
          }
          // row maximum of the half: four independent chains of 3-input max
          float mx4[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t* sp = &s[q >> 1][(q & 1) * 16];
            float m = fmaxf(__uint_as_float(sp[0]), __uint_as_float(sp[1]));
#pragma unroll
            for (int i = 2; i < 16; i += 2) m = fmax3(m, __uint_as_float(sp[i]), __uint_as_float(sp[i + 1]));
            mx4[q] = m;
          }
          // running maximum m_cur is kept in log2 units (raw maximum * cj)
          constexpr float kBias = QK8 ? 12582912.f : 0.f;
          float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          if constexpr (QK8) mx -= kBias;
          mx *= cj;
          float alpha = 1.f;
          if (j == 0 && hb == 0) {
            m_cur = mx;
          } else {
            const float m_new = fmaxf(m_cur, mx);
            if (m_new - m_cur > kLazyThreshold) {  // also taken when m_cur = -inf
              alpha = ex2(m_cur - m_new);
              m_cur = m_new;
            }
          }
          alpha_smem[(2 * t + hb) * kTileM + r] = alpha;
          warp_arrive(bar(L::kBarAlpha + 2 * t + hb));
          if (t == 0 && j == 0 && hb == 0) warp_arrive(bar(L::kBarStagger));

          // exponent of a score x: x*cj - m; for the int8 variant x carries kBias, taken out here
          float mc = (m_cur == -INFINITY) ? 0.f : m_cur;
          if constexpr (QK8) mc = fmaf(kBias, cj, mc);
          // two scores per FMA / ADD issue slot (packed f32x2); the exp2 itself is one per lane,
          // except that one pair in eight (one in four at D = 64, where the exp2 unit is the
          // bound) is evaluated by a polynomial on the FMA pipe: the exp2 unit (16 results per
          // clock per SM) is co-critical with the tensor pipe, the FMA pipe has room.  Larger
          // shares measured slower (3/8 and 1/2: the issue slots run out).
          constexpr int kPolyMask = (D == 64) ? 7 : 15;
          uint64_t psum = pack_f32x2(0.f, 0.f);
          const uint64_t cj2 = pack_f32x2(cj, cj), mc2 = pack_f32x2(-mc, -mc);
          uint32_t pk[32];
#pragma unroll
          for (int q = 0; q < 2; ++q)
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float x0, x1;
              unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[q][i]), __uint_as_float(s[q][i + 1])), cj2, mc2),
                           x0, x1);
              float p0, p1;
              if ((i & kPolyMask) == 0) {
                exp2_poly_f32x2(x0, x1, p0, p1);
              } else {
                p0 = ex2(x0);
                p1 = ex2(x1);
              }
              psum = add_f32x2(psum, pack_f32x2(p0, p1));
              pk[q * 16 + (i >> 1)] = pack2<BF16>(p0, p1);
            }
          float psum0, psum1;
          unpack_f32x2(psum, psum0, psum1);
          l_run = l_run * alpha + (psum0 + psum1);
          tmem_st32(tS + hb * kHalfN, pk);  // P of this half over the first 32 columns of its S
          tmem_wait_st();
          tc_fence_before();
          warp_arrive(bar(L::kBarPReady + 2 * t + hb));
        }
      }

      if ((!PLAN || pe_nparts == 1) && !(CARRY && a.carry_mode != 0) && a.lse != nullptr && row < a.Nq) {
        const float lse = (l_run > 0.f) ? (m_cur * 0.6931471805599453f + __logf(l_run)) : -INFINITY;
        a.lse[(static_cast<long long>(b) * a.Hq + h) * a.Nq + row] = lse;
      }
      const uint32_t tO = tmem_base + L::kColO + D * t + lane_off;
      if (n_tiles > 0) {
        mbar_wait(bar(L::kBarODone + 2 * t + 1), (n_tiles - 1) & 1, wc, kErrWaitO);
        tc_fence_after();
      }
      // A CTA that covers a piece of an item's key range publishes its partial result; the last
      // piece to arrive folds the other pieces into its own accumulator and writes the output.
      // factor of this CTA's own accumulator; a row that never saw a visible key (running maximum
      // still -inf) yields zeros even though its masked scores left 2^-126 terms in l_run (the
      // polynomial exp2 clamps its argument)
      float f_self = (l_run > 0.f && m_cur != -INFINITY) ? (1.f / l_run) : 0.f;
      float f_part = 0.f;            // factor of the partial waiting in shared memory (if any)
      const float4* s_part = nullptr; // that partial: [D/4][128 rows][4] fp32, offset to this row
      bool write_out = true;
      if constexpr (PLAN) {
        if (pe_nparts > 1) {
          // Count in first.  The piece that arrives last keeps its result in TMEM and merges; the
          // others publish theirs: un-normalised O as [D/4][128 rows][4] fp32 (a warp writes 512
          // contiguous bytes per store) and (m, l) of every row, then count themselves published.
          int* cnt = a.counters + 4 * pe_counter + 2 * t;  // [0] arrived, [1] published
          if (r == 0) arrival[t] = atomicAdd(cnt, 1);
          named_bar_sync(kBarEpilogue + t, 128);
          write_out = (arrival[t] == pe_nparts - 1);
          if (!write_out) {
            const long long my = (static_cast<long long>(pe_slot0 + pe_part) * 2 + t) * kTileM;
            float4* po = reinterpret_cast<float4*>(a.part_o + my * D) + r;
#pragma unroll
            for (int q = 0; q < D / 32; ++q) {
              uint32_t o[32];
              tmem_ld32(tO + q * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int g = 0; g < 8; ++g)
                po[(q * 8 + g) * kTileM] =
                    make_float4(__uint_as_float(o[4 * g]), __uint_as_float(o[4 * g + 1]),
                                __uint_as_float(o[4 * g + 2]), __uint_as_float(o[4 * g + 3]));
            }
            a.part_ml[my + r] = make_float2(m_cur, l_run);
            __threadfence();
            named_bar_sync(kBarEpilogue + t, 128);
            if (r == 0) {
              __threadfence();  // release: the group's stores (ordered by the barrier) before the count
              atomicAdd(cnt + 1, 1);
            }
          } else {
            // Every other piece has counted in, so it is publishing right now or has finished:
            // a short, bounded wait for the last of them, then the counters go back to zero.
            if (r == 0) {
              count_wait(cnt + 1, pe_nparts - 1, wc, kErrWaitPeer);
              __threadfence();  // acquire side: nothing below is read before the count was seen
              cnt[0] = 0;
              cnt[1] = 0;
            }
            named_bar_sync(kBarEpilogue + t, 128);
            __threadfence();
            // The other pieces' partials come in through the K/V ring (this tile's half of it),
            // one bulk copy each; the ring is free once the other Q tile's MMAs are done too.
            // The first copy is started before anything else so that the rest overlaps it.
            if (nt == 2) mbar_wait(bar(L::kBarODone + 2 * (1 - t) + 1), (n_tiles - 1) & 1, wc, kErrWaitO);
            constexpr uint32_t kPartBytes = D * kTileM * 4;
            const uint32_t ring_off = L::kOffRing + t * (L::kStages / 2) * L::kTileBytes;
            const int first_other = (pe_part == 0) ? 1 : 0;
            const int last_other = (pe_part == pe_nparts - 1) ? pe_nparts - 2 : pe_nparts - 1;
            auto fetch = [&](int p) {
              mbar_expect_tx(bar(L::kBarQFull + t), kPartBytes);
              bulk_load(sbase + ring_off, a.part_o + (static_cast<long long>(pe_slot0 + p) * 2 + t) * kTileM * D,
                        kPartBytes, bar(L::kBarQFull + t));
            };
            if (r == 0) {
              fence_proxy_async_all();
              fetch(first_other);
            }
            // totals of the row over all pieces, one pass (the same running-maximum rule)
            const float2* ml0 = a.part_ml + (static_cast<long long>(pe_slot0) * 2 + t) * kTileM + r;
            float m_tot = m_cur, l_tot = l_run, m_first = -INFINITY;
#pragma unroll 4
            for (int p = 0; p < pe_nparts; ++p) {
              if (p == pe_part) continue;
              const float2 ml = __ldcg(ml0 + static_cast<long long>(p) * 2 * kTileM);
              if (p == first_other) m_first = ml.x;
              const float m_new = fmaxf(m_tot, ml.x);
              const float mn = (m_new == -INFINITY) ? 0.f : m_new;
              l_tot = l_tot * ex2(m_tot - mn) + ml.y * ex2(ml.x - mn);
              m_tot = m_new;
            }
            const float mt = (m_tot == -INFINITY) ? 0.f : m_tot;
            const float inv_l = (l_tot > 0.f) ? (1.f / l_tot) : 0.f;
            if (a.lse != nullptr && row < a.Nq)
              a.lse[(static_cast<long long>(b) * a.Hq + h) * a.Nq + row] =
                  (l_tot > 0.f) ? (m_tot * 0.6931471805599453f + __logf(l_tot)) : -INFINITY;
            s_part = reinterpret_cast<const float4*>(gbase + ring_off) + r;
            uint32_t phase = 1;  // the Q barrier of this tile completed its phase 0 with the Q load
            bool own_scaled = false;
            const float w_self = ex2(m_cur - mt);
            for (int p = 0; p < pe_nparts; ++p) {
              if (p == pe_part) continue;
              if (p != first_other && r == 0) fetch(p);
              const float m_p = (p == first_other) ? m_first : __ldcg(ml0 + static_cast<long long>(p) * 2 * kTileM).x;
              const float wp = ex2(m_p - mt);
              mbar_wait(bar(L::kBarQFull + t), phase, wc, kErrWaitKV);
              phase ^= 1;
              if (p == last_other) {  // folded in while the output is written, below
                f_part = wp * inv_l;
                break;
              }
              // more than two pieces: accumulate into the TMEM accumulator
#pragma unroll
              for (int q = 0; q < D / 32; ++q) {
                uint32_t o[32];
                tmem_ld32(tO + q * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                  const float4 x = s_part[(q * 8 + g) * kTileM];
                  const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float own = own_scaled ? __uint_as_float(o[4 * g + e]) : __uint_as_float(o[4 * g + e]) * w_self;
                    o[4 * g + e] = __float_as_uint(fmaf(xs[e], wp, own));
                  }
                }
                tmem_st32(tO + q * 32, o);
              }
              tmem_wait_st();
              own_scaled = true;
              named_bar_sync(kBarEpilogue + t, 128);  // everyone has read the partial: the next may land
            }
            f_self = own_scaled ? inv_l : w_self * inv_l;
          }
        }
      }
      if constexpr (CARRY) {
        if (a.carry_mode != 0) {
          const long long tix =
              (static_cast<long long>(b) * a.Hq + h) * a.carry_tiles + a.carry_tile0 + (q0 / kTileM + t);
          float* c_o = a.carry_o + tix * kTileM * D;
          float2* c_ml = a.carry_ml + tix * kTileM;
          constexpr uint32_t kPartBytes = D * kTileM * 4;
          const uint32_t ring_off = L::kOffRing + t * (L::kStages / 2) * L::kTileBytes;
          float m_tot = m_cur, l_tot = l_run, w_self = 1.f, w_c = 0.f;
          if (a.carry_mode & 1) {
            // The state comes in through this tile's half of the K/V ring, idle once the other
            // Q tile's MMAs are done too.
            if (n_tiles > 0 && nt == 2)
              mbar_wait(bar(L::kBarODone + 2 * (1 - t) + 1), (n_tiles - 1) & 1, wc, kErrWaitO);
            if (r == 0) {
              fence_proxy_async_all();
              mbar_expect_tx(bar(L::kBarQFull + t), kPartBytes);
              bulk_load(sbase + ring_off, c_o, kPartBytes, bar(L::kBarQFull + t));
            }
            const float2 ml = __ldcg(c_ml + r);
            m_tot = fmaxf(m_cur, ml.x);
            const float mt = (m_tot == -INFINITY) ? 0.f : m_tot;
            w_self = ex2(m_cur - mt);
            w_c = ex2(ml.x - mt);
            l_tot = l_run * w_self + ml.y * w_c;
            // the tile's Q barrier completed phase 0 with the Q load (issued only when there are keys)
            mbar_wait(bar(L::kBarQFull + t), n_tiles > 0 ? 1u : 0u, wc, kErrWaitKV);
            s_part = reinterpret_cast<const float4*>(gbase + ring_off) + r;
          }
          if (a.carry_mode & 2) {
            // new state: O relative to the merged maximum, still un-normalised
            write_out = false;
            float4* po = reinterpret_cast<float4*>(c_o) + r;
#pragma unroll
            for (int q = 0; q < D / 32; ++q) {
              uint32_t o[32];
              if (n_tiles > 0) {
                tmem_ld32(tO + q * 32, o);
                tmem_wait_ld();
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = 0u;
              }
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                float4 x = make_float4(__uint_as_float(o[4 * g]) * w_self, __uint_as_float(o[4 * g + 1]) * w_self,
                                       __uint_as_float(o[4 * g + 2]) * w_self, __uint_as_float(o[4 * g + 3]) * w_self);
                if (s_part != nullptr) {
                  const float4 y = s_part[(q * 8 + g) * kTileM];
                  x.x = fmaf(y.x, w_c, x.x);
                  x.y = fmaf(y.y, w_c, x.y);
                  x.z = fmaf(y.z, w_c, x.z);
                  x.w = fmaf(y.w, w_c, x.w);
                }
                po[(q * 8 + g) * kTileM] = x;
              }
            }
            c_ml[r] = make_float2(m_tot, l_tot);
          } else {
            const float inv_l = (l_tot > 0.f) ? (1.f / l_tot) : 0.f;
            f_self = w_self * inv_l;
            f_part = w_c * inv_l;
            if (a.lse != nullptr && row < a.Nq)
              a.lse[(static_cast<long long>(b) * a.Hq + h) * a.Nq + row] =
                  (l_tot > 0.f) ? (m_tot * 0.6931471805599453f + __logf(l_tot)) : -INFINITY;
          }
        }
      }
      if (write_out) {
        // ---- epilogue of this Q tile (the two softmax groups run theirs side by side):
        //      O / l -> 16 bit -> swizzled smem (the tile's Q buffer) -> TMA store
        const uint32_t stage = sQ + t * L::kTileBytes;
#pragma unroll
        for (int q = 0; q < D / 32; ++q) {
          float o[32];
          if (n_tiles > 0) {
            uint32_t u[32];
            tmem_ld32(tO + q * 32, u);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(u[i]) * f_self;
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0.f;
          }
          if constexpr (PLAN || CARRY) {
            if (s_part != nullptr) {
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                const float4 x = s_part[(q * 8 + g) * kTileM];
                o[4 * g + 0] = fmaf(x.x, f_part, o[4 * g + 0]);
                o[4 * g + 1] = fmaf(x.y, f_part, o[4 * g + 1]);
                o[4 * g + 2] = fmaf(x.z, f_part, o[4 * g + 2]);
                o[4 * g + 3] = fmaf(x.w, f_part, o[4 * g + 3]);
              }
            }
          }
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            const int col = q * 32 + ch * 8;
            const int bx = col >> 6;
            const int chunk = (col & 63) >> 3;
            const uint32_t addr = stage + bx * kBoxBytes + r * 128 + ((chunk ^ (r & 7)) << 4);
            const uint32_t w0 = pack2<BF16>(o[ch * 8 + 0], o[ch * 8 + 1]);
            const uint32_t w1 = pack2<BF16>(o[ch * 8 + 2], o[ch * 8 + 3]);
            const uint32_t w2 = pack2<BF16>(o[ch * 8 + 4], o[ch * 8 + 5]);
            const uint32_t w3 = pack2<BF16>(o[ch * 8 + 6], o[ch * 8 + 7]);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w0), "r"(w1),
                         "r"(w2), "r"(w3)
                         : "memory");
          }
        }
        fence_proxy_async_smem();
        named_bar_sync(kBarEpilogue + t, 128);
        if (r == 0) {
#pragma unroll
          for (int bx = 0; bx < L::kBoxes; ++bx)
            tma_store_4d(&tm_o, stage + bx * kBoxBytes, bx * kBoxCols, q0 + t * kTileM, h, b);
          tma_store_commit();
          tma_store_wait_read0();  // the staging buffer must outlive the copy's reads, no more
        }
      }
      tc_fence_before();
    }
  } else if (warp < 12) {
    // =========================== correction ========================================
    reg_dec<kRegCorr>();
    const int r = tid & 127;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    for (int j = 0; j < n_tiles; ++j) {
#pragma unroll
      for (int hb = 0; hb < 2; ++hb) {
        for (int t = 0; t < nt; ++t) {
          mbar_wait(bar(L::kBarAlpha + 2 * t + hb), j & 1, wc, kErrWaitCorr);
          const float alpha = alpha_smem[(2 * t + hb) * kTileM + r];
          if ((j > 0 || hb > 0) && __any_sync(0xffffffffu, alpha != 1.f)) {
            // every PV issued so far into O_t must have finished: the previous half-step's
            if (hb == 0) mbar_wait(bar(L::kBarODone + 2 * t + 1), (j - 1) & 1, wc, kErrWaitO);
            else mbar_wait(bar(L::kBarODone + 2 * t + 0), j & 1, wc, kErrWaitO);
            tc_fence_after();
            const uint32_t tO = tmem_base + L::kColO + D * t + lane_off;
#pragma unroll
            for (int q = 0; q < D / 32; ++q) {
              uint32_t o[32];
              tmem_ld32(tO + q * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(tO + q * 32, o);
            }
            tmem_wait_st();
            tc_fence_before();
          }
          warp_arrive(bar(L::kBarOReady + 2 * t + hb));
        }
      }
    }
    tc_fence_before();
  } else {
    reg_dec<kRegOther>();
    if (warp == 12 || warp == 14) {
      // =========================== MMA issuers =====================================
      // One issuing thread per Q tile (warp 12 -> tile 0, warp 14 -> tile 1).  Each walks its
      // tile's halves in the order the softmax group publishes them: PV_a(j) S_a(j+1) PV_b(j)
      // S_b(j+1).  The tensor pipe interleaves the two streams.
      const int t = (warp == 12) ? 0 : 1;
      if (lane == 0 && n_tiles > 0 && t < nt) {
        // kind::f16: D fmt f32, A/B f16 or bf16.  kind::i8: D fmt s32 (2), A/B signed int8 (1).
        constexpr uint32_t idesc_s =
            QK8 ? make_idesc(2, 1, 0, 0, kTileM, kHalfN) : make_idesc(1, BF16 ? 1 : 0, 0, 0, kTileM, kHalfN);
        constexpr uint32_t idesc_o = make_idesc(1, BF16 ? 1 : 0, 0, 1, kTileM, D);
        const uint32_t sQt = sQ + t * L::kTileBytes;
        const uint32_t tO = tmem_base + L::kColO + D * t;
        const uint32_t tSt = tmem_base + L::kColS + 128 * t;
        // S(half) = Q_t . K[64*half .. 64*half+64)^T  ->  TMEM columns [128t + 64half, +64)
        auto issue_s = [&](int hb, int slot) {
          const uint32_t d_tmem = tSt + kHalfN * hb;
          if constexpr (QK8) {
            // The accumulator starts at 1.5*2^23 in every element: one fp16 MMA of two constant
            // tiles (3072 * 4096 in the k = 0 term, zeros elsewhere) writes the fp32 bit pattern
            // 0x4B400000, and the int8 MMAs then add the integer dot products onto those bits.
            // The softmax reads the words as the floats 12582912 + acc.
            constexpr uint32_t idesc_bias = make_idesc(1, 0, 0, 0, kTileM, kHalfN);
            mma_f16_ss(d_tmem, make_smem_desc(sbase + L::kOffBiasA, 16, 1024),
                       make_smem_desc(sbase + L::kOffBiasB, 16, 1024), idesc_bias, 0u);
            // int8 rows are D bytes: 64-byte swizzle (8 rows = 512 B) at D=64, 128-byte at D=128;
            // one MMA consumes K = 32 bytes.
            constexpr uint32_t kLayout = (D == 64) ? 4u : 2u;
            constexpr uint32_t kSbo = (D == 64) ? 512u : 1024u;
            const uint32_t kb = sRing + slot * L::kTileBytes + hb * kHalfN * D;
#pragma unroll
            for (int k = 0; k < D / 32; ++k) {
              const uint64_t da = make_smem_desc(sQt + k * 32, 16, kSbo, kLayout);
              const uint64_t db = make_smem_desc(kb + k * 32, 16, kSbo, kLayout);
              mma_i8_ss(d_tmem, da, db, idesc_s, 1u);
            }
          } else {
            const uint32_t kb = sRing + slot * L::kTileBytes + hb * kHalfN * 128;
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
              const uint32_t off = (k / 4) * kBoxBytes + (k % 4) * 32;
              const uint64_t da = make_smem_desc(sQt + off, 16, 1024);
              const uint64_t db = make_smem_desc(kb + off, 16, 1024);
              mma_f16_ss(d_tmem, da, db, idesc_s, k > 0);
            }
          }
        };
        mbar_wait(bar(L::kBarQFull + t), 0, wc, kErrWaitKV);
        int cons = 0;  // ring consumption index: K_0, V_0, K_1, V_1, ...
        mbar_wait(bar(L::kBarKvFull + 0), 0, wc, kErrWaitKV);
        // Start tile 1 about half a softmax step after tile 0 (when tile 0 has published its
        // first row maxima): the two softmax groups then alternate between their max and exp2
        // phases instead of competing for the exp2 unit at the same moments.  The barrier
        // completes exactly once, so a late issuer can never mistake a later phase for it.
        if (t == 1) mbar_wait(bar(L::kBarStagger), 0, wc, kErrWaitP);
        tc_fence_after();
        for (int hb = 0; hb < 2; ++hb) {
          issue_s(hb, 0);
          mma_commit(bar(L::kBarSFull + 2 * t + hb));
        }
        mma_commit(bar(L::kBarKvEmpty + 0));
        cons = 1;
        for (int j = 0; j < n_tiles; ++j) {
          const int vslot = cons % L::kStages;
          mbar_wait(bar(L::kBarKvFull + vslot), (cons / L::kStages) & 1, wc, kErrWaitKV);
          ++cons;
          const bool has_next = (j + 1 < n_tiles);
          const int kslot = cons % L::kStages;
          const uint32_t kpar = (cons / L::kStages) & 1;
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) {
            mbar_wait(bar(L::kBarOReady + 2 * t + hb), j & 1, wc, kErrWaitCorr);
            mbar_wait(bar(L::kBarPReady + 2 * t + hb), j & 1, wc, kErrWaitP);
            tc_fence_after();
            const uint32_t tP = tSt + kHalfN * hb;
#pragma unroll
            for (int kk = 0; kk < kHalfN / 16; ++kk) {
              const int k = hb * (kHalfN / 16) + kk;  // 16-key slice of the V tile
              const uint64_t db =
                  make_smem_desc(sRing + vslot * L::kTileBytes + k * 2048, kBoxBytes, 1024);
              mma_f16_ts(tO, tP + kk * 8, db, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
            }
            mma_commit(bar(L::kBarODone + 2 * t + hb));
            if (hb == 1) mma_commit(bar(L::kBarKvEmpty + vslot));
            if (has_next) {  // S_h(j+1) after PV_h(j), whose operand P_h(j) lives in the S buffer
              if (hb == 0) {
                mbar_wait(bar(L::kBarKvFull + kslot), kpar, wc, kErrWaitKV);
                tc_fence_after();
              }
              issue_s(hb, kslot);
              mma_commit(bar(L::kBarSFull + 2 * t + hb));
              if (hb == 1) mma_commit(bar(L::kBarKvEmpty + kslot));
            }
          }
          if (has_next) ++cons;
        }
      }
      __syncwarp();
    } else if (warp == 13) {
      // =========================== TMA producer ====================================
      if (lane == 0 && n_tiles > 0) {
        for (int i = n_early; i < n_fill; ++i) {
          const int slot = i % L::kStages;
          const int use = i / L::kStages;
          mbar_wait(bar(L::kBarKvEmpty + slot), (use - 1) & 1, wc, kErrWaitFree);
          load_kv(i);
        }
        // On the give-up path copies may still be in flight: let them land (bounded)
        // before the CTA's shared memory is released.
        if (*abort_flag) {
          const uint64_t t0 = global_timer_ns();
          while (global_timer_ns() - t0 < 2000000ull) {
          }
        }
      }
      __syncwarp();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 12) {
    tc_fence_after();
    tmem_dealloc(tmem_base, L::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------
// The opt-in to more than 48 KB of dynamic shared memory is per function and per device; it is
// made once for each (the reference does it at import, flash_attention.cu:140-147), not on every
// launch.  `done` holds one bit per device ordinal.
template <typename Kernel>
static cudaError_t allow_dynamic_smem(Kernel kern, int bytes, std::atomic<unsigned long long>* done) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const bool tracked = dev >= 0 && dev < 64;
  if (tracked && ((done->load(std::memory_order_acquire) >> dev) & 1ull)) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && tracked) done->fetch_or(1ull << dev, std::memory_order_release);
  return e;
}

template <int D, bool BF16, bool QK8, bool CARRY = false>
static cudaError_t launch_ws_t(const CUtensorMap* tm, const FwdArgs& a, int sm_count, cudaStream_t st) {
  using L = WsLayout<D, QK8>;
  auto kern = fwd_ws_kernel<D, BF16, QK8, false, CARRY>;
  static std::atomic<unsigned long long> smem_set{0};  // per instantiation: devices already configured
  cudaError_t e = allow_dynamic_smem(kern, L::kDynSmem, &smem_set);
  if (e != cudaSuccess) return e;
  const long long n_pairs = (a.n_q_tiles + 1) / 2;
  const long long items = n_pairs * a.Hq * a.B;
  if (items > 0x7fffffffll) return cudaErrorInvalidValue;
  // One CTA per SM: `items` CTAs run in ceil(items / SMs) waves.  When the last (or only) wave
  // would be at most half full, its pairs are split into single-tile CTAs (twice as many, each
  // shorter), which still fit one wave; needs every tile to be real (even tile count) and enough
  // K/V tiles to amortise a CTA (measured: a gain from 4 tiles on).
  FwdArgs args = a;
  args.n_pair_items = static_cast<int>(items);
  args.part_o = nullptr;
  args.part_ml = nullptr;
  args.counters = nullptr;
  long long grid = items;
  const long long rest = sm_count > 0 ? items % sm_count : 0;
  const long long kv_tiles = (a.Nk + kTileN - 1) / kTileN;
  if (rest > 0 && 2 * rest <= sm_count && (a.n_q_tiles % 2) == 0 && (kv_tiles >= 8 || (items < sm_count && kv_tiles >= 4))) {
    args.n_pair_items = static_cast<int>(items - rest);
    grid = items + rest;
  }
  kern<<<static_cast<unsigned>(grid), kNumThreads, L::kDynSmem, st>>>(tm[0], tm[1], tm[2], tm[3],
                                                                      args, NoPlanTable{0});
  return cudaGetLastError();
}

template <int D, bool BF16, bool QK8>
static cudaError_t launch_plan_t(const CUtensorMap* tm, const FwdArgs& a, const FwdPlan& plan,
                                 cudaStream_t st) {
  using L = WsLayout<D, QK8>;
  auto kern = fwd_ws_kernel<D, BF16, QK8, true>;
  static std::atomic<unsigned long long> smem_set{0};
  cudaError_t e = allow_dynamic_smem(kern, L::kDynSmem, &smem_set);
  if (e != cudaSuccess) return e;
  FwdArgs args = a;
  args.n_pair_items = plan.n_whole;
  const unsigned grid = static_cast<unsigned>(plan.n_whole + plan.n_table);
  kern<<<grid, kNumThreads, L::kDynSmem, st>>>(tm[0], tm[1], tm[2], tm[3], args, plan.table);
  return cudaGetLastError();
}

// Balanced launch: a.part_o / a.part_ml / a.counters point into the caller's scratch.  qk8: the
// INT8-QK variant (tm[0], tm[1] are the int8 Q / K maps).
cudaError_t launch_fwd_ws_plan(int D, bool bf16, bool qk8, const CUtensorMap* tm, const FwdArgs& a,
                               const FwdPlan& plan, cudaStream_t st) {
  if (D == 128) {
    if (qk8) return bf16 ? launch_plan_t<128, true, true>(tm, a, plan, st) : launch_plan_t<128, false, true>(tm, a, plan, st);
    return bf16 ? launch_plan_t<128, true, false>(tm, a, plan, st) : launch_plan_t<128, false, false>(tm, a, plan, st);
  }
  if (D == 64) {
    if (qk8) return bf16 ? launch_plan_t<64, true, true>(tm, a, plan, st) : launch_plan_t<64, false, true>(tm, a, plan, st);
    return bf16 ? launch_plan_t<64, true, false>(tm, a, plan, st) : launch_plan_t<64, false, false>(tm, a, plan, st);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_fwd_ws(int D, bool bf16, const CUtensorMap* tm, const FwdArgs& a, int sm_count,
                          cudaStream_t st) {
  if (a.carry_mode != 0) {  // a ring step: running state in, state or output out
    if (D == 128)
      return bf16 ? launch_ws_t<128, true, false, true>(tm, a, sm_count, st)
                  : launch_ws_t<128, false, false, true>(tm, a, sm_count, st);
    if (D == 64)
      return bf16 ? launch_ws_t<64, true, false, true>(tm, a, sm_count, st)
                  : launch_ws_t<64, false, false, true>(tm, a, sm_count, st);
    return cudaErrorInvalidValue;
  }
  if (D == 128)
    return bf16 ? launch_ws_t<128, true, false>(tm, a, sm_count, st) : launch_ws_t<128, false, false>(tm, a, sm_count, st);
  if (D == 64)
    return bf16 ? launch_ws_t<64, true, false>(tm, a, sm_count, st) : launch_ws_t<64, false, false>(tm, a, sm_count, st);
  return cudaErrorInvalidValue;
}

// tm[0], tm[1]: int8 Q / K maps (one box of D bytes x 128 rows); tm[2], tm[3]: 16-bit V / O maps.
cudaError_t launch_fwd_ws_int8qk(int D, bool bf16, const CUtensorMap* tm, const FwdArgs& a,
                                 int sm_count, cudaStream_t st) {
  if (D == 128)
    return bf16 ? launch_ws_t<128, true, true>(tm, a, sm_count, st) : launch_ws_t<128, false, true>(tm, a, sm_count, st);
  if (D == 64)
    return bf16 ? launch_ws_t<64, true, true>(tm, a, sm_count, st) : launch_ws_t<64, false, true>(tm, a, sm_count, st);
  return cudaErrorInvalidValue;
}

}  // namespace ma
