// INT8 pre-pass for the INT8-QK attention variant (no counterpart in the reference code; the
// recipe is the SageAttention-style one of the task configuration):
//   1. K is smoothed: the per-(batch, KV head, channel) mean over tokens is subtracted.  Every
//      score of a row moves by the same amount q.mean(K), so softmax is unchanged.
//   2. Q and the smoothed K are quantised to int8 with one symmetric fp32 scale per block of 128
//      tokens: scale = max|x| / 127 over the 128 x D slab (1 for an all-zero slab),
//      x8 = round-half-even(x / scale), clamped to [-127, 127].
// Two launches: stage 1 quantises Q and sums the columns of K (independent work, one grid), stage 2
// smooths and quantises K.  Stage 2 is launched as a programmatic dependent of stage 1: its CTAs
// become resident while stage 1 drains and load their K slabs before they wait for stage 1's
// column sums, so the second launch's ramp and first loads hide under the first one's tail.
// HBM-bound byte movers: 16-byte loads, 8-byte int8 stores, one CTA per
// (128-token block, head, batch) or per 1024-token column-sum chunk.  Algorithmic traffic per element: K 2 B (mean pass) + 2 B + 1 B,
// Q 2 B + 1 B, plus 4 B per 128 x D slab for the scale.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

namespace ma {

// Scratch of the allocation-free pre-pass entry point (miniattn_quant_qk_int8_static): the
// column sums of K, B * Hkv * ceil(Nk/1024) * D floats, at most kStaticColsumFloats (256 KB).
// Every GPU that loads the library holds this array until the process exits.  In host code the
// name below is only a handle for cudaGetSymbolAddress, never a device address.
constexpr long long kStaticColsumFloats = 65536;
static __device__ __align__(256) float g_static_colsum[kStaticColsumFloats];

namespace {

template <bool BF16>
__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]) {
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 a;
    if constexpr (BF16) {
      a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u[i]));
    } else {
      a = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
    }
    f[2 * i] = a.x;
    f[2 * i + 1] = a.y;
  }
}

constexpr int kSumRows = 1024;  // tokens per partial column sum

}  // namespace

// partial[b, h, chunk, d] = sum over the chunk's tokens of k[b, h, token, d]
template <int D, bool BF16>
__device__ __forceinline__ void colsum_body(const uint16_t* __restrict__ k, long long sb, long long sh,
                                            long long sn, int N, float* __restrict__ partial,
                                            int n_chunks, int chunk, int h, int b, int H) {
  constexpr int CPR = D / 8;          // 16-byte chunks per row
  constexpr int RPP = 256 / CPR;      // rows per pass
  const int col8 = threadIdx.x % CPR, r0 = threadIdx.x / CPR;
  const uint16_t* base = k + b * sb + h * sh;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const int row_end = min(N, (chunk + 1) * kSumRows);
  for (int row = chunk * kSumRows + r0; row < row_end; row += RPP) {
    const uint4 w = *reinterpret_cast<const uint4*>(base + row * sn + col8 * 8);
    float f[8];
    unpack8<BF16>(w, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += f[i];
  }
  __shared__ float red[RPP][D];
#pragma unroll
  for (int i = 0; i < 8; ++i) red[r0][col8 * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < D) {
    float s = 0.f;
#pragma unroll 4
    for (int r = 0; r < RPP; ++r) s += red[r][threadIdx.x];
    partial[((static_cast<long long>(b) * H + h) * n_chunks + chunk) * D + threadIdx.x] = s;
  }
}

// One CTA per (128-token block, head, batch): x8 = round(x' / scale), x' = x - mean (K) or x (Q).
template <int D, bool BF16, bool SMOOTH>
__device__ __forceinline__ void quant_body(const uint16_t* __restrict__ x, long long sb, long long sh,
                                           long long sn, int N, const float* __restrict__ partial,
                                           int n_chunks, int8_t* __restrict__ x8,
                                           float* __restrict__ scale_out, float fold,
                                           float* __restrict__ mean_out, int blk, int h, int b, int H,
                                           int n_blocks) {
  constexpr int CPR = D / 8;
  constexpr int PER = 16 * D / 256;  // chunks per thread (128 rows * D/8 chunks / 256 threads)
  __shared__ float mean[D];
  __shared__ float wmax[8];
  const uint16_t* base = x + b * sb + h * sh;
  // The slab stays in registers as loaded (16-bit pairs) and is unpacked twice, once for the
  // maximum and once for the quantisation: a quarter of the registers of an fp32 copy, so more
  // CTAs (and bytes in flight) fit an SM.  The loads are issued before the channel means are
  // summed, so that the two global-memory latencies overlap.
  uint4 raw[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int id = threadIdx.x + i * 256;
    const int row = blk * 128 + id / CPR, col8 = id % CPR;
    raw[i] = make_uint4(0u, 0u, 0u, 0u);
    if (row < N) raw[i] = *reinterpret_cast<const uint4*>(base + row * sn + col8 * 8);
  }
  if (SMOOTH) {
    // everything above is independent of stage 1; its column sums are complete and visible from here
    cudaGridDependencySynchronize();
    if (threadIdx.x < D) {
      float s = 0.f;
      const float* p = partial + (static_cast<long long>(b) * H + h) * n_chunks * D + threadIdx.x;
      for (int c = 0; c < n_chunks; ++c) s += p[c * D];
      const float m = s / static_cast<float>(N);
      mean[threadIdx.x] = m;
      if (blk == 0 && mean_out != nullptr) mean_out[(static_cast<long long>(b) * H + h) * D + threadIdx.x] = m;
    }
    __syncthreads();
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int id = threadIdx.x + i * 256;
    const int row = blk * 128 + id / CPR, col8 = id % CPR;
    if (row < N) {
      float f[8];
      unpack8<BF16>(raw[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (SMOOTH) f[e] -= mean[col8 * 8 + e];
        amax = fmaxf(amax, fabsf(f[e]));
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = wmax[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, wmax[w]);
  const float scale = amax > 0.f ? __fdiv_rn(amax, 127.f) : 1.f;
  const float inv = __frcp_rn(scale);
  if (threadIdx.x == 0)
    scale_out[(static_cast<long long>(b) * H + h) * n_blocks + blk] = scale * fold;
  int8_t* obase = x8 + ((static_cast<long long>(b) * H + h) * N) * D;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int id = threadIdx.x + i * 256;
    const int row = blk * 128 + id / CPR, col8 = id % CPR;
    if (row < N) {
      float f[8];
      unpack8<BF16>(raw[i], f);
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (SMOOTH) f[e] -= mean[col8 * 8 + e];
        // round-half-even(x / scale), bit for bit, without a division per element: y = x * (1/scale)
        // is within 2e-5 of the true quotient, and adding 1.5*2^23 rounds it to the nearest integer
        // (ties to even) in the low mantissa bits.  Only when y lies within 1e-3 of a tie can the
        // two roundings differ; those elements (about 0.2 %) take the exact division.
        const float y = f[e] * inv;
        const float t = y + 12582912.f;
        const float d = y - (t - 12582912.f);
        int qv;
        if (fabsf(d) > 0.499f) {
          qv = __float2int_rn(__fdiv_rn(f[e], scale));
          qv = max(-127, min(127, qv));
        } else {
          qv = __float_as_int(t) - 0x4B400000;
        }
        if (e < 4) lo |= (static_cast<uint32_t>(qv) & 0xFFu) << (8 * e);
        else hi |= (static_cast<uint32_t>(qv) & 0xFFu) << (8 * (e - 4));
      }
      *reinterpret_cast<uint2*>(obase + static_cast<long long>(row) * D + col8 * 8) = make_uint2(lo, hi);
    }
  }
}

// Stage 1, one launch: the Q quantiser (nothing depends on it but the attention kernel) and the
// partial column sums of K.  The first gridDim.x - q_blocks blocks sum K, the rest quantise Q.
template <int D, bool BF16>
__global__ void __launch_bounds__(256)
prepass_stage1_kernel(const uint16_t* __restrict__ q, long long qsb, long long qsh, long long qsn, int Nq,
                      int Hq, int nqb, int8_t* __restrict__ q8, float* __restrict__ sq, float fold,
                      const uint16_t* __restrict__ k, long long ksb, long long ksh, long long ksn, int Nk,
                      int Hkv, int nch, float* __restrict__ partial, int q_blocks) {
  // the dependent launch (stage 2) may start as soon as every CTA of this grid is under way
  cudaTriggerProgrammaticLaunchCompletion();
  // the column-sum CTAs read eight times as much as a quantiser CTA: they go first
  const int s_blocks = static_cast<int>(gridDim.x) - q_blocks;
  if (static_cast<int>(blockIdx.x) >= s_blocks) {
    const int id = blockIdx.x - s_blocks;
    const int blk = id % nqb, h = (id / nqb) % Hq, b = id / (nqb * Hq);
    quant_body<D, BF16, false>(q, qsb, qsh, qsn, Nq, nullptr, 0, q8, sq, fold, nullptr, blk, h, b, Hq, nqb);
  } else {
    const int c = blockIdx.x;
    const int chunk = c % nch, h = (c / nch) % Hkv, b = c / (nch * Hkv);
    colsum_body<D, BF16>(k, ksb, ksh, ksn, Nk, partial, nch, chunk, h, b, Hkv);
  }
}

// Stage 2: smooth and quantise K (needs every column sum of stage 1).
template <int D, bool BF16>
__global__ void __launch_bounds__(256)
quant_k_kernel(const uint16_t* __restrict__ k, long long sb, long long sh, long long sn, int N,
               const float* __restrict__ partial, int n_chunks, int8_t* __restrict__ k8,
               float* __restrict__ scale_out, float* __restrict__ mean_out) {
  quant_body<D, BF16, true>(k, sb, sh, sn, N, partial, n_chunks, k8, scale_out, 1.0f, mean_out,
                            blockIdx.x, blockIdx.y, blockIdx.z, gridDim.y, gridDim.x);
}

// q8/k8: contiguous [B, H, N, D] int8; scales: [B, H, ceil(N/128)] fp32; partial: scratch of
// B * Hkv * ceil(N/1024) * D floats; k_mean (optional): [B, Hkv, D].
template <int D, bool BF16>
static cudaError_t launch_quant_t(const void* q, const long long* qs, const void* k, const long long* ks,
                                  int B, int Hq, int Hkv, int Nq, int Nk, float q_fold, int8_t* q8,
                                  int8_t* k8, float* sq, float* sk, float* partial, float* k_mean,
                                  cudaStream_t st) {
  const int nqb = (Nq + 127) / 128, nkb = (Nk + 127) / 128, nch = (Nk + kSumRows - 1) / kSumRows;
  const long long q_blocks = static_cast<long long>(nqb) * Hq * B;
  const long long s_blocks = static_cast<long long>(nch) * Hkv * B;
  if (q_blocks + s_blocks > 0x7fffffffll) return cudaErrorInvalidValue;
  if (q_blocks + s_blocks > 0)
    prepass_stage1_kernel<D, BF16><<<static_cast<unsigned>(q_blocks + s_blocks), 256, 0, st>>>(
        static_cast<const uint16_t*>(q), qs[0], qs[1], qs[2], Nq, Hq, nqb, q8, sq, q_fold,
        static_cast<const uint16_t*>(k), ks[0], ks[1], ks[2], Nk, Hkv, nch, partial, static_cast<int>(q_blocks));
  if (Nk > 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nkb, Hkv, B);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (q_blocks + s_blocks > 0) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, quant_k_kernel<D, BF16>, static_cast<const uint16_t*>(k), ks[0], ks[1],
                                       ks[2], Nk, static_cast<const float*>(partial), nch, k8, sk, k_mean);
    if (e != cudaSuccess) return e;
  }
  return cudaGetLastError();
}

cudaError_t launch_quant_qk(int D, bool bf16, const void* q, const long long* qs, const void* k,
                            const long long* ks, int B, int Hq, int Hkv, int Nq, int Nk, float q_fold,
                            int8_t* q8, int8_t* k8, float* sq, float* sk, float* partial, float* k_mean,
                            cudaStream_t st) {
  if (D == 64)
    return bf16 ? launch_quant_t<64, true>(q, qs, k, ks, B, Hq, Hkv, Nq, Nk, q_fold, q8, k8, sq, sk, partial, k_mean, st)
                : launch_quant_t<64, false>(q, qs, k, ks, B, Hq, Hkv, Nq, Nk, q_fold, q8, k8, sq, sk, partial, k_mean, st);
  if (D == 128)
    return bf16 ? launch_quant_t<128, true>(q, qs, k, ks, B, Hq, Hkv, Nq, Nk, q_fold, q8, k8, sq, sk, partial, k_mean, st)
                : launch_quant_t<128, false>(q, qs, k, ks, B, Hq, Hkv, Nq, Nk, q_fold, q8, k8, sq, sk, partial, k_mean, st);
  return cudaErrorInvalidValue;
}

long long static_colsum_capacity() { return kStaticColsumFloats; }

// Device address of g_static_colsum on the current device, looked up once per device with that
// device current (the first call on a device does the lookup).
static cudaError_t static_colsum_ptr(float** out) {
  static std::mutex mu;
  static float* ptrs[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_colsum);
    if (e != cudaSuccess) return e;
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return cudaSuccess;
}

// Same pre-pass as launch_quant_qk with the column-sum scratch taken from g_static_colsum.
// Nothing in the array has to start at zero: the column-sum kernel overwrites every entry the
// quantiser reads.  The caller has checked that the problem fits kStaticColsumFloats.
cudaError_t launch_quant_qk_static(int D, bool bf16, const void* q, const long long* qs, const void* k,
                                   const long long* ks, int B, int Hq, int Hkv, int Nq, int Nk,
                                   float q_fold, int8_t* q8, int8_t* k8, float* sq, float* sk,
                                   float* k_mean, cudaStream_t st) {
  float* scratch = nullptr;
  cudaError_t e = static_colsum_ptr(&scratch);
  if (e != cudaSuccess) return e;
  return launch_quant_qk(D, bf16, q, qs, k, ks, B, Hq, Hkv, Nq, Nk, q_fold, q8, k8, sq, sk, scratch,
                         k_mean, st);
}

}  // namespace ma
