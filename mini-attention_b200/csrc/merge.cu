// Log-sum-exp merge of attention partials (ring / context-parallel mode).
//
// A ring step yields, for every query row, a normalised partial output o_p (16 bit) over the
// keys of the visiting K/V chunk and lse_p = ln(sum exp) over those keys.  The running result
// (o_acc fp32, lse_acc) is updated as
//     m = max(lse_acc, lse_p);  wa = e^(lse_acc-m);  wb = e^(lse_p-m)
//     o_acc = (o_acc*wa + o_p*wb) / (wa+wb);   lse_acc = m + ln(wa+wb)
// which is the split-KV merge of the reference's decode benchmark
// (kernels/standard/pytorch/benchmark_mla_decode_torch.py:244-272) applied pairwise.
// An lse of -inf marks an empty partial (no visible key).  HBM-bound: one warp per row,
// 16-byte accesses, algorithmic traffic per row = D*(4+2+4) bytes (+2*D when `out` is written).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace ma {

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (BF16) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&w));
  }
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack2f(float a, float b) {
  if constexpr (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

// D = 32 * VEC elements per row; VEC = 4 (D=128) or 2 (D=64)
template <int VEC, bool BF16>
__global__ void __launch_bounds__(256)
merge_partials_kernel(float* __restrict__ acc_o, float* __restrict__ acc_lse,
                      const uint16_t* __restrict__ part_o, const float* __restrict__ part_lse,
                      uint16_t* __restrict__ out, long long rows, int init, long long rows_per_slab,
                      long long out_slab_stride) {
  constexpr int D = 32 * VEC;
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; row < rows;
       row += warps) {
    const float lp = part_lse[row];
    float p[VEC];
    if constexpr (VEC == 4) {
      const uint2 w = *reinterpret_cast<const uint2*>(part_o + row * D + lane * 4);
      const float2 a = unpack2<BF16>(w.x), b = unpack2<BF16>(w.y);
      p[0] = a.x; p[1] = a.y; p[2] = b.x; p[3] = b.y;
    } else {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(part_o + row * D + lane * 2);
      const float2 a = unpack2<BF16>(w);
      p[0] = a.x; p[1] = a.y;
    }
    float r[VEC];
    float lse_new;
    if (init) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) r[i] = p[i];
      lse_new = lp;
    } else {
      const float la = acc_lse[row];
      float o[VEC];
      if constexpr (VEC == 4) {
        const float4 v = *reinterpret_cast<const float4*>(acc_o + row * D + lane * 4);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
      } else {
        const float2 v = *reinterpret_cast<const float2*>(acc_o + row * D + lane * 2);
        o[0] = v.x; o[1] = v.y;
      }
      const float m = fmaxf(la, lp);
      const float ms = (m == -INFINITY) ? 0.f : m;
      const float wa = __expf(la - ms), wb = __expf(lp - ms);
      const float den = wa + wb;
      const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) r[i] = (o[i] * wa + p[i] * wb) * inv;
      lse_new = den > 0.f ? ms + __logf(den) : -INFINITY;
    }
    if constexpr (VEC == 4) {
      *reinterpret_cast<float4*>(acc_o + row * D + lane * 4) = make_float4(r[0], r[1], r[2], r[3]);
    } else {
      *reinterpret_cast<float2*>(acc_o + row * D + lane * 2) = make_float2(r[0], r[1]);
    }
    if (lane == 0) acc_lse[row] = lse_new;
    if (out != nullptr) {
      // `out` may be a token-range view of a larger tensor: slabs of rows_per_slab rows (one
      // (batch, head) each) lie out_slab_stride elements apart
      uint16_t* orow = out + (row / rows_per_slab) * out_slab_stride + (row % rows_per_slab) * D;
      if constexpr (VEC == 4) {
        uint2 w;
        w.x = pack2f<BF16>(r[0], r[1]);
        w.y = pack2f<BF16>(r[2], r[3]);
        *reinterpret_cast<uint2*>(orow + lane * 4) = w;
      } else {
        *reinterpret_cast<uint32_t*>(orow + lane * 2) = pack2f<BF16>(r[0], r[1]);
      }
    }
  }
}

cudaError_t launch_merge_partials(float* acc_o, float* acc_lse, const void* part_o,
                                  const float* part_lse, void* out, long long rows, int D, bool bf16,
                                  int init, long long rows_per_slab, long long out_slab_stride,
                                  int sm_count, cudaStream_t st) {
  if (rows == 0) return cudaSuccess;
  const long long blocks_needed = (rows + 7) / 8;  // 8 warps (rows) per 256-thread block
  const long long cap = static_cast<long long>(sm_count) * 8;  // grid: multiple of the SM count
  const unsigned grid = static_cast<unsigned>(blocks_needed < cap ? blocks_needed : cap);
  const uint16_t* po = static_cast<const uint16_t*>(part_o);
  uint16_t* oo = static_cast<uint16_t*>(out);
  if (D == 128) {
    if (bf16) merge_partials_kernel<4, true><<<grid, 256, 0, st>>>(acc_o, acc_lse, po, part_lse, oo, rows, init, rows_per_slab, out_slab_stride);
    else merge_partials_kernel<4, false><<<grid, 256, 0, st>>>(acc_o, acc_lse, po, part_lse, oo, rows, init, rows_per_slab, out_slab_stride);
  } else if (D == 64) {
    if (bf16) merge_partials_kernel<2, true><<<grid, 256, 0, st>>>(acc_o, acc_lse, po, part_lse, oo, rows, init, rows_per_slab, out_slab_stride);
    else merge_partials_kernel<2, false><<<grid, 256, 0, st>>>(acc_o, acc_lse, po, part_lse, oo, rows, init, rows_per_slab, out_slab_stride);
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace ma
