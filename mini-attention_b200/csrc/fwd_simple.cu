// Forward attention, "simple" sm_100a kernel: one 128-row Q tile per CTA, 128 threads,
// no role specialisation.  It exists to pin down the TMA / tcgen05 / TMEM plumbing
// (descriptors, swizzled layouts, barrier protocol) with the least moving parts and is
// the fallback the warp-specialised kernel is checked against.
//
// Same math as the reference mainloop (kernels/flash_attn/cuda/sm_120/kernel/include/
// forward_kernel.cuh:137-221): per K/V tile S = Q K^T (fp32), online softmax in the
// exp2 domain (softmax.cuh:29-107), O += P V (fp32), final O / l.
//
// Per CTA and K/V tile:
//   thread 0 : TMA K_j,V_j (two-slot ring) ; 8x tcgen05.mma S = Q K_j^T -> TMEM[0,128)
//   all      : tcgen05.ld S row (thread = row) ; max / exp2 / sum ; rescale O in TMEM ;
//              P (16-bit) -> 128B-swizzled smem
//   thread 0 : 8x tcgen05.mma O += P V_j -> TMEM[128,128+D)  (V consumed MN-major)
// Epilogue   : O / l -> 16 bit -> swizzled smem -> TMA store (rows past Nq are clipped).
#include "common.cuh"
#include "ptx.cuh"

namespace ma {

template <int D>
struct SimpleLayout {
  static constexpr int kBoxes = D / kBoxCols;            // 64-column boxes per tile
  static constexpr int kTileBytes = kBoxes * kBoxBytes;  // one Q / K / V tile
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kOffQ + kTileBytes;       // 2 slots
  static constexpr int kOffV = kOffK + 2 * kTileBytes;   // 2 slots
  static constexpr int kOffP = kOffV + 2 * kTileBytes;   // 128 x 128 x 2 B
  static constexpr int kOffBar = kOffP + 2 * kBoxBytes;
  static constexpr int kBytes = kOffBar + 128;
  static constexpr int kDynSmem = kBytes + 1024;         // slack for 1024-B alignment
  static constexpr int kTmemCols = 256;                  // S: [0,128)  O: [128,128+D)
};

template <int D, bool BF16>
__global__ void __launch_bounds__(128, 1)
fwd_simple_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                  const FwdArgs a) {
  using L = SimpleLayout<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (sbase - raw);

  const uint32_t sQ = sbase + L::kOffQ;
  const uint32_t sK = sbase + L::kOffK;
  const uint32_t sV = sbase + L::kOffV;
  const uint32_t sP = sbase + L::kOffP;
  const uint32_t bar_q = sbase + L::kOffBar;
  const uint32_t bar_kv0 = bar_q + 8;   // two slots: +8, +16
  const uint32_t bar_s = bar_q + 24;
  const uint32_t bar_o = bar_q + 32;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + L::kOffBar + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + L::kOffBar + 72);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (a.Hq / a.Hkv);
  const int q0 = qt * kTileM;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_kv0, 1);
    mbar_init(bar_kv0 + 8, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
    prefetch_tmap(&tm_o);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), L::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;
  const uint32_t tmem_O = tmem_base + 128;
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
  const WaitCtx wc{abort_flag, a.status, MINIATTN_WAIT_LIMIT_NS};

  // number of K/V tiles this Q tile has to visit
  int kv_end = a.Nk;
  if (a.causal) {
    const int last_row = min(q0 + kTileM - 1, a.Nq - 1);
    const long long vis = a.q_pos0 + last_row - a.k_pos0 + 1;  // keys [0, vis) visible to it
    kv_end = static_cast<int>(max(0ll, min(static_cast<long long>(a.Nk), vis)));
  }
  const int n_tiles = (kv_end + kTileN - 1) / kTileN;

  // keys [0, vis_row) are visible to this thread's query row
  const int row = q0 + tid;
  long long vis_row_ll = a.Nk;
  if (a.causal) vis_row_ll = min(vis_row_ll, a.q_pos0 + row - a.k_pos0 + 1);
  const int vis_row = static_cast<int>(max(0ll, vis_row_ll));

  constexpr uint32_t idesc_s = make_idesc(1, BF16 ? 1 : 0, 0, 0, kTileM, kTileN);
  constexpr uint32_t idesc_o = make_idesc(1, BF16 ? 1 : 0, 0, 1, kTileM, D);

  auto load_kv = [&](int j, int slot) {
    const uint32_t bar = bar_kv0 + 8 * slot;
    mbar_expect_tx(bar, 2 * L::kTileBytes);
#pragma unroll
    for (int bx = 0; bx < L::kBoxes; ++bx) {
      tma_load_4d(sK + slot * L::kTileBytes + bx * kBoxBytes, &tm_k, bar, bx * kBoxCols,
                  j * kTileN, hk, b);
      tma_load_4d(sV + slot * L::kTileBytes + bx * kBoxBytes, &tm_v, bar, bx * kBoxCols,
                  j * kTileN, hk, b);
    }
  };

  if (tid == 0 && n_tiles > 0) {
    mbar_expect_tx(bar_q, L::kTileBytes);
#pragma unroll
    for (int bx = 0; bx < L::kBoxes; ++bx)
      tma_load_4d(sQ + bx * kBoxBytes, &tm_q, bar_q, bx * kBoxCols, q0, h, b);
    load_kv(0, 0);
  }

  float m_run = -INFINITY;  // running max of raw scores
  float l_run = 0.f;        // running sum of exp
  const float c = a.scale_log2;

  for (int j = 0; j < n_tiles; ++j) {
    const int slot = j & 1;
    if (tid == 0) {
      if (j + 1 < n_tiles) load_kv(j + 1, slot ^ 1);
      if (j == 0) mbar_wait(bar_q, 0, wc, kErrWaitKV);
      mbar_wait(bar_kv0 + 8 * slot, (j >> 1) & 1, wc, kErrWaitKV);
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < D / 16; ++k) {
        const uint32_t off = (k / 4) * kBoxBytes + (k % 4) * 32;
        const uint64_t da = make_smem_desc(sQ + off, 16, 1024);
        const uint64_t db = make_smem_desc(sK + slot * L::kTileBytes + off, 16, 1024);
        mma_f16_ss(tmem_S, da, db, idesc_s, k > 0);
      }
      mma_commit(bar_s);
    }
    __syncwarp();
    mbar_wait(bar_s, j & 1, wc, kErrWaitS);
    tc_fence_after();

    // ---- S row -> registers -------------------------------------------------
    uint32_t sreg[4][32];
#pragma unroll
    for (int q = 0; q < 4; ++q) tmem_ld32(tmem_S + lane_off + q * 32, sreg[q]);
    tmem_wait_ld();

    const int lim = vis_row - j * kTileN;  // keys [0, lim) of this tile are visible
    float mx = -INFINITY;
    if (lim >= kTileN) {
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sreg[q][i]));
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (q * 32 + i >= lim) sreg[q][i] = __float_as_uint(-INFINITY);
          mx = fmaxf(mx, __uint_as_float(sreg[q][i]));
        }
    }
    const float m_new = fmaxf(m_run, mx);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = ex2((m_run - m_use) * c);  // m_run = -inf -> 0
    const float mc = m_use * c;
    float psum = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float p = ex2(fmaf(__uint_as_float(sreg[q][i]), c, -mc));
        psum += p;
        sreg[q][i] = __float_as_uint(p);
      }
    l_run = l_run * alpha + psum;
    m_run = m_new;

    // ---- P -> swizzled smem (K-major A operand of the PV MMA) ------------------
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {  // 8 columns = one 16-byte chunk
        const int col = q * 32 + ch * 8;
        const int bx = col >> 6;
        const int chunk = (col & 63) >> 3;
        const uint32_t addr = sP + bx * kBoxBytes + tid * 128 + ((chunk ^ (tid & 7)) << 4);
        const uint32_t w0 = pack2<BF16>(__uint_as_float(sreg[q][ch * 8 + 0]),
                                        __uint_as_float(sreg[q][ch * 8 + 1]));
        const uint32_t w1 = pack2<BF16>(__uint_as_float(sreg[q][ch * 8 + 2]),
                                        __uint_as_float(sreg[q][ch * 8 + 3]));
        const uint32_t w2 = pack2<BF16>(__uint_as_float(sreg[q][ch * 8 + 4]),
                                        __uint_as_float(sreg[q][ch * 8 + 5]));
        const uint32_t w3 = pack2<BF16>(__uint_as_float(sreg[q][ch * 8 + 6]),
                                        __uint_as_float(sreg[q][ch * 8 + 7]));
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w0), "r"(w1),
                     "r"(w2), "r"(w3)
                     : "memory");
      }
    }

    // ---- rescale the O accumulator in TMEM -------------------------------------
    if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
      for (int q = 0; q < D / 32; ++q) {
        uint32_t o[32];
        tmem_ld32(tmem_O + lane_off + q * 32, o);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st32(tmem_O + lane_off + q * 32, o);
      }
      tmem_wait_st();
    }

    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < kTileN / 16; ++k) {
        const uint64_t da =
            make_smem_desc(sP + (k / 4) * kBoxBytes + (k % 4) * 32, 16, 1024);
        const uint64_t db =
            make_smem_desc(sV + slot * L::kTileBytes + k * 2048, kBoxBytes, 1024);
        mma_f16_ss(tmem_O, da, db, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
      }
      mma_commit(bar_o);
    }
    __syncwarp();
    mbar_wait(bar_o, j & 1, wc, kErrWaitO);
    tc_fence_after();
  }

  // ---- epilogue: O / l -> 16 bit -> swizzled smem (Q's buffer) -> TMA store ------
  const float inv_l = (l_run > 0.f) ? (1.f / l_run) : 0.f;
#pragma unroll
  for (int q = 0; q < D / 32; ++q) {
    uint32_t o[32];
    if (n_tiles > 0) {
      tmem_ld32(tmem_O + lane_off + q * 32, o);
      tmem_wait_ld();
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) o[i] = 0u;
    }
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      const int col = q * 32 + ch * 8;
      const int bx = col >> 6;
      const int chunk = (col & 63) >> 3;
      const uint32_t addr = sQ + bx * kBoxBytes + tid * 128 + ((chunk ^ (tid & 7)) << 4);
      const uint32_t w0 = pack2<BF16>(__uint_as_float(o[ch * 8 + 0]) * inv_l,
                                      __uint_as_float(o[ch * 8 + 1]) * inv_l);
      const uint32_t w1 = pack2<BF16>(__uint_as_float(o[ch * 8 + 2]) * inv_l,
                                      __uint_as_float(o[ch * 8 + 3]) * inv_l);
      const uint32_t w2 = pack2<BF16>(__uint_as_float(o[ch * 8 + 4]) * inv_l,
                                      __uint_as_float(o[ch * 8 + 5]) * inv_l);
      const uint32_t w3 = pack2<BF16>(__uint_as_float(o[ch * 8 + 6]) * inv_l,
                                      __uint_as_float(o[ch * 8 + 7]) * inv_l);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w0), "r"(w1),
                   "r"(w2), "r"(w3)
                   : "memory");
    }
  }
  if (a.lse != nullptr && row < a.Nq) {
    const float lse = (l_run > 0.f) ? (m_run * a.scale + __logf(l_run)) : -INFINITY;
    a.lse[(static_cast<long long>(b) * a.Hq + h) * a.Nq + row] = lse;
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
#pragma unroll
    for (int bx = 0; bx < L::kBoxes; ++bx)
      tma_store_4d(&tm_o, sQ + bx * kBoxBytes, bx * kBoxCols, q0, h, b);
    tma_store_commit();
    tma_store_wait_all();
    // On the give-up path a K/V copy may still be in flight: let it land (bounded)
    // before the CTA's shared memory is released.
    if (*abort_flag) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) {
      }
    }
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, L::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------
template <int D, bool BF16>
static cudaError_t launch_simple_t(const CUtensorMap* tm, const FwdArgs& a, cudaStream_t st) {
  using L = SimpleLayout<D>;
  auto kern = fwd_simple_kernel<D, BF16>;
  cudaError_t e =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynSmem);
  if (e != cudaSuccess) return e;
  dim3 grid(a.n_q_tiles, a.Hq, a.B);
  kern<<<grid, 128, L::kDynSmem, st>>>(tm[0], tm[1], tm[2], tm[3], a);
  return cudaGetLastError();
}

cudaError_t launch_fwd_simple(int D, bool bf16, const CUtensorMap* tm, const FwdArgs& a,
                              cudaStream_t st) {
  if (D == 128) return bf16 ? launch_simple_t<128, true>(tm, a, st) : launch_simple_t<128, false>(tm, a, st);
  if (D == 64) return bf16 ? launch_simple_t<64, true>(tm, a, st) : launch_simple_t<64, false>(tm, a, st);
  return cudaErrorInvalidValue;
}

}  // namespace ma
