// Host side of the C ABI declared in include/miniattn.h: argument validation
// (mirrors the checks of the reference launcher, kernels/flash_attn/cuda/sm_120/kernel/
// flash_attention.cu:41-80, relaxed to "head dim contiguous" instead of fully contiguous),
// TMA tensor-map construction from the caller's strides, kernel selection and launch.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <vector>

#include "../../include/miniattn.h"
#include "common.cuh"

namespace ma {
cudaError_t launch_fwd_simple(int D, bool bf16, const CUtensorMap* tm, const FwdArgs& a,
                              cudaStream_t st);
cudaError_t launch_fwd_ws(int D, bool bf16, const CUtensorMap* tm, const FwdArgs& a, int sm_count,
                          cudaStream_t st);
cudaError_t launch_fwd_ws_int8qk(int D, bool bf16, const CUtensorMap* tm, const FwdArgs& a,
                                 int sm_count, cudaStream_t st);
cudaError_t launch_fwd_ws_plan(int D, bool bf16, bool qk8, const CUtensorMap* tm, const FwdArgs& a,
                               const FwdPlan& plan, cudaStream_t st);
void plan_fwd(const FwdArgs& a, int D, int sms, FwdPlan* plan);
cudaError_t launch_quant_qk(int D, bool bf16, const void* q, const long long* qs, const void* k,
                            const long long* ks, int B, int Hq, int Hkv, int Nq, int Nk, float q_fold,
                            int8_t* q8, int8_t* k8, float* sq, float* sk, float* partial, float* k_mean,
                            cudaStream_t st);
long long static_colsum_capacity();
cudaError_t launch_quant_qk_static(int D, bool bf16, const void* q, const long long* qs, const void* k,
                                   const long long* ks, int B, int Hq, int Hkv, int Nq, int Nk,
                                   float q_fold, int8_t* q8, int8_t* k8, float* sq, float* sk,
                                   float* k_mean, cudaStream_t st);
cudaError_t launch_wait_selftest(int32_t* status, unsigned long long limit_ns, cudaStream_t st);
cudaError_t launch_merge_partials(float* acc_o, float* acc_lse, const void* part_o,
                                  const float* part_lse, void* out, long long rows, int D, bool bf16,
                                  int init, long long rows_per_slab, long long out_slab_stride,
                                  int sm_count, cudaStream_t st);
}  // namespace ma

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 4-D map over a [B, H, N, D] logical tensor with arbitrary (batch, head, token) strides:
// dims (fastest first) = (d, token, head, batch); box = 64 x `box_rows` x 1 x 1 elements
// (one 128-byte swizzled row per token).
// Recently encoded maps of the calling thread: a loop that calls the operator on the same tensors
// pays the driver's encoder once (four encodes are about a third of the host time of a launch).
struct MapKey {
  const void* base;
  int64_t stride[3];
  int elem_bytes, dt, D, N, H, B, box_cols, box_rows, swizzle;
  bool operator==(const MapKey& o) const {
    return base == o.base && stride[0] == o.stride[0] && stride[1] == o.stride[1] && stride[2] == o.stride[2] &&
           elem_bytes == o.elem_bytes && dt == o.dt && D == o.D && N == o.N && H == o.H && B == o.B &&
           box_cols == o.box_cols && box_rows == o.box_rows && swizzle == o.swizzle;
  }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool valid;
};
constexpr int kMapSlots = 16;

int make_map(CUtensorMap* out, const void* base, int elem_bytes, CUtensorMapDataType dt, int D,
             int N, int H, int B, const int64_t stride[3], int box_cols, int box_rows,
             const char* what, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  thread_local MapSlot cache[kMapSlots] = {};
  thread_local unsigned next_slot = 0;
  const MapKey key{base, {stride[0], stride[1], stride[2]}, elem_bytes, static_cast<int>(dt), D, N, H, B,
                   box_cols, box_rows, static_cast<int>(swizzle)};
  for (int i = 0; i < kMapSlots; ++i)
    if (cache[i].valid && cache[i].key == key) {
      *out = cache[i].map;
      return MINIATTN_OK;
    }
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fail(MINIATTN_ECUDA, "cuTensorMapEncodeTiled entry point not found");
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)stride[2] * elem_bytes, (cuuint64_t)stride[1] * elem_bytes,
                           (cuuint64_t)stride[0] * elem_bytes};
  cuuint32_t box[4] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  // a size-1 dim may carry any stride; give the encoder a legal one
  for (int i = 0; i < 3; ++i)
    if (dims[i + 1] == 1) strides[i] = (cuuint64_t)D * elem_bytes;
  CUresult r = enc(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MINIATTN_ECUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
  MapSlot& slot = cache[next_slot++ % kMapSlots];
  slot.key = key;
  slot.map = *out;
  slot.valid = true;
  return MINIATTN_OK;
}

int check_tensor(const void* p, const int64_t s[3], int D, const char* name) {
  if (p == nullptr) return fail(MINIATTN_EINVAL, "%s is null", name);
  if (reinterpret_cast<uintptr_t>(p) % 16 != 0)
    return fail(MINIATTN_EINVAL, "%s must be 16-byte aligned", name);
  for (int i = 0; i < 3; ++i) {
    if (s[i] < 0) return fail(MINIATTN_EINVAL, "%s has a negative stride", name);
    if (s[i] % 8 != 0)
      return fail(MINIATTN_EINVAL, "%s stride %d (%lld) is not a multiple of 8 elements", name, i,
                  (long long)s[i]);
  }
  if (s[2] < D) return fail(MINIATTN_EINVAL, "%s token stride is smaller than D", name);
  return MINIATTN_OK;
}

int device_sm_count(int* sms, int* major) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(MINIATTN_ECUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  // one entry per device ordinal, filled on first use under a lock (host threads may drive
  // different devices at the same time)
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static int table_sms[kMaxDevices] = {0};
  static int table_major[kMaxDevices] = {0};
  if (dev < 0 || dev >= kMaxDevices) return fail(MINIATTN_EUNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> g(mu);
  if (table_sms[dev] == 0) {
    int n = 0, mj = 0;
    if ((e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&mj, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess)
      return fail(MINIATTN_ECUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
    table_sms[dev] = n;
    table_major[dev] = mj;
  }
  *sms = table_sms[dev];
  *major = table_major[dev];
  return MINIATTN_OK;
}

}  // namespace

extern "C" {

const char* miniattn_version(void) { return "miniattn-b200 0.2 sm_100a"; }

// Head dim the kernels are instantiated for.  D = 96 runs on the D = 128 kernels: the tensor maps
// carry the true extent, so TMA zero-fills columns 96..127 of every Q, K and V tile on the way in
// (zeros change neither Q K^T nor P V) and clips them from the O tile on the way out.
static int kernel_head_dim(int D) { return D == 96 ? 128 : D; }

const char* miniattn_last_error_string(void) { return g_err; }

// Shared argument checks of the forward entry points.  Returns 1 when there is nothing to do.
static int check_fwd_params(const MiniAttnFwdParams* p) {
  if (p == nullptr) return fail(MINIATTN_EINVAL, "params is null");
  if (p->dtype != MINIATTN_FP16 && p->dtype != MINIATTN_BF16)
    return fail(MINIATTN_EUNSUPPORTED, "dtype must be fp16 (0) or bf16 (1), got %d", p->dtype);
  if (p->D != 64 && p->D != 96 && p->D != 128)
    return fail(MINIATTN_EUNSUPPORTED, "head dim %d not supported (64, 96 or 128)", p->D);
  if (p->B < 0 || p->Hq < 0 || p->Hkv < 0 || p->Nq < 0 || p->Nk < 0)
    return fail(MINIATTN_EINVAL, "negative size");
  if (p->B == 0 || p->Hq == 0 || p->Nq == 0) return 1;  // empty output: nothing to do
  if (p->Hkv == 0 || p->Hq % p->Hkv != 0)
    return fail(MINIATTN_EINVAL, "Hq (%d) must be a positive multiple of Hkv (%d)", p->Hq, p->Hkv);
  if (p->Hq > 65535 || p->B > 65535)
    return fail(MINIATTN_EUNSUPPORTED, "B and Hq must not exceed 65535");
  if (p->causal != 0 && p->causal != 1) return fail(MINIATTN_EINVAL, "causal must be 0 or 1");
  if (p->kernel < MINIATTN_KERNEL_AUTO || p->kernel > MINIATTN_KERNEL_WS)
    return fail(MINIATTN_EINVAL, "unknown kernel selector %d", p->kernel);
  if ((p->carry_in != 0 && p->carry_in != 1) || (p->carry_out != 0 && p->carry_out != 1))
    return fail(MINIATTN_EINVAL, "carry_in and carry_out must be 0 or 1");
  const bool carry = p->carry_in || p->carry_out;
  if (carry) {
    if (p->carry == nullptr) return fail(MINIATTN_EINVAL, "carry_in / carry_out set but carry is null");
    if (reinterpret_cast<uintptr_t>(p->carry) % 256 != 0)
      return fail(MINIATTN_EINVAL, "carry must be 256-byte aligned");
    if (p->kernel == MINIATTN_KERNEL_SIMPLE)
      return fail(MINIATTN_EUNSUPPORTED, "the carried state needs the warp-specialised kernel");
    const int tiles = (p->Nq + ma::kTileM - 1) / ma::kTileM;
    if (p->carry_tile0 < 0 || p->carry_tiles < 0 ||
        (p->carry_tiles == 0 ? p->carry_tile0 != 0 : p->carry_tile0 + tiles > p->carry_tiles))
      return fail(MINIATTN_EINVAL, "carry_tile0 (%d) + the %d Q tiles of this call exceed carry_tiles (%d)",
                  p->carry_tile0, tiles, p->carry_tiles);
  }
  int rc;
  if ((rc = check_tensor(p->q, p->q_stride, p->D, "q")) != 0) return rc;
  // a call that only stores the running state writes no output: o may be null then
  if (!(p->carry_out && p->o == nullptr) && (rc = check_tensor(p->o, p->o_stride, p->D, "o")) != 0) return rc;
  // With no keys every row is fully masked; K/V pointers are still handed to the tensor-map
  // encoder, so they must be valid whenever Nk > 0.
  const bool has_keys = p->Nk > 0;
  if (has_keys) {
    if ((rc = check_tensor(p->k, p->k_stride, p->D, "k")) != 0) return rc;
    if ((rc = check_tensor(p->v, p->v_stride, p->D, "v")) != 0) return rc;
  }

  return MINIATTN_OK;
}

// Group size of the work-item order (FwdArgs::bh_group).  When the K and V of all heads together
// exceed what L2 keeps of them (its 126 MB are two partitions, and Q and O stream through as well),
// walking all heads at once makes every wave of CTAs fetch K and V from HBM again: measured on a
// 16384 x 16384 task with 32 heads, 7.6 GB of DRAM reads for 0.4 GB of operands.  Groups whose K/V
// fit a share of L2 bring that back to about one read.  A group is a whole number of KV heads
// (with the query heads they serve) and divides B*Hq.
#ifndef MINIATTN_GROUP_TOTAL_MB
#define MINIATTN_GROUP_TOTAL_MB 48
#define MINIATTN_GROUP_SHARE_MB 40
#endif
static int head_group(const MiniAttnFwdParams* p) {
  const long long bh_total = static_cast<long long>(p->B) * p->Hq;
  if (p->Hkv <= 0 || p->Hq % p->Hkv != 0) return static_cast<int>(bh_total > 0 ? bh_total : 1);
  const long long g = p->Hq / p->Hkv;                               // query heads per KV head
  const long long kv_heads = static_cast<long long>(p->B) * p->Hkv;
  const long long per_kv = 2ll * p->Nk * kernel_head_dim(p->D) * 2; // K and V bytes of one KV head
  if (per_kv * kv_heads < (static_cast<long long>(MINIATTN_GROUP_TOTAL_MB) << 20)) return static_cast<int>(bh_total);
  long long want = (static_cast<long long>(MINIATTN_GROUP_SHARE_MB) << 20) / (per_kv > 0 ? per_kv : 1);
  if (want < 1) want = 1;
  long long d = 1;
  for (long long c = 1; c <= want && c <= kv_heads; ++c)
    if (kv_heads % c == 0) d = c;
  return static_cast<int>(d * g);
}

static void fill_args(const MiniAttnFwdParams* p, ma::FwdArgs* a) {
  a->lse = p->lse;
  a->status = p->status;
  a->q_pos0 = p->q_pos0;
  a->k_pos0 = p->k_pos0;
  a->Nq = p->Nq;
  a->Nk = p->Nk;
  a->Hq = p->Hq;
  a->Hkv = p->Hkv;
  a->B = p->B;
  a->causal = p->causal;
  a->scale = p->softmax_scale > 0.f ? p->softmax_scale : 1.0f / sqrtf((float)p->D);
  a->scale_log2 = a->scale * 1.4426950408889634f;
  a->n_q_tiles = (p->Nq + ma::kTileM - 1) / ma::kTileM;
  a->n_pair_items = 0;  // set by the warp-specialised launcher
  a->bh_group = head_group(p);
  a->sq = nullptr;
  a->sk = nullptr;
  a->part_o = nullptr;
  a->part_ml = nullptr;
  a->counters = nullptr;
  a->carry_o = nullptr;
  a->carry_ml = nullptr;
  a->carry_mode = 0;
  a->carry_tile0 = 0;
  a->carry_tiles = 0;
}

static int check_device(int* sms) {
  int major = 0, rc;
  if ((rc = device_sm_count(sms, &major)) != 0) return rc;
  if (major != 10)
    return fail(MINIATTN_EUNSUPPORTED,
                "this library holds sm_100a code only; current device has compute capability %d.x",
                major);
  return MINIATTN_OK;
}

// Plans of recent shapes (planning costs up to a millisecond of host time; launches of one shape
// repeat).  Guarded by a mutex; an entry is copied out under the lock.
namespace {
struct PlanKey {
  int Nq, Nk, B, Hq, causal, D, sms, group;
  long long diag;
  bool operator==(const PlanKey& o) const {
    return Nq == o.Nq && Nk == o.Nk && B == o.B && Hq == o.Hq && causal == o.causal && D == o.D &&
           sms == o.sms && group == o.group && diag == o.diag;
  }
};
struct PlanSlot {
  PlanKey key;
  std::shared_ptr<const ma::FwdPlan> plan;
};
std::shared_ptr<const ma::FwdPlan> cached_plan(const ma::FwdArgs& a, int D, int sms) {
  static std::mutex mu;
  static std::vector<PlanSlot> cache;
  static size_t next = 0;
  const PlanKey key{a.Nq, a.Nk, a.B, a.Hq, a.causal, D, sms, a.bh_group, a.causal ? a.q_pos0 - a.k_pos0 : 0};
  {
    std::lock_guard<std::mutex> g(mu);
    for (const PlanSlot& s : cache)
      if (s.key == key) return s.plan;
  }
  auto plan = std::make_shared<ma::FwdPlan>();
  ma::plan_fwd(a, D, sms, plan.get());
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() < 16) cache.push_back(PlanSlot{key, plan});
  else cache[next++ % 16] = PlanSlot{key, plan};
  return plan;
}

constexpr size_t kCounterBytes = 16384;  // (arrived, published) x 2 Q tiles x kPlanCap cut items, rounded up
static_assert(4 * ma::kPlanCap * sizeof(int) <= kCounterBytes, "counter region too small");
size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }
size_t scratch_bytes_of(const ma::FwdPlan& plan, int D) {
  if (!plan.split) return 0;
  const size_t rows = static_cast<size_t>(plan.n_slots) * 2 * ma::kTileM;
  return kCounterBytes + align256(rows * sizeof(float2)) + rows * D * sizeof(float);
}
}  // namespace

// Points the kernel arguments at the three regions of a balanced launch's scratch.
static int bind_scratch(const ma::FwdPlan& plan, int D, void* scratch, size_t scratch_bytes, ma::FwdArgs* a) {
  const size_t need = scratch_bytes_of(plan, D);
  if (scratch_bytes < need)
    return fail(MINIATTN_EINVAL, "scratch holds %zu bytes, this launch needs %zu "
                "(miniattn_fwd_balanced_scratch_bytes)", scratch_bytes, need);
  if (reinterpret_cast<uintptr_t>(scratch) % 256 != 0)
    return fail(MINIATTN_EINVAL, "scratch must be 256-byte aligned");
  uint8_t* base = static_cast<uint8_t*>(scratch);
  const size_t rows = static_cast<size_t>(plan.n_slots) * 2 * ma::kTileM;
  a->counters = reinterpret_cast<int*>(base);
  a->part_ml = reinterpret_cast<float2*>(base + kCounterBytes);
  a->part_o = reinterpret_cast<float*>(base + kCounterBytes + align256(rows * sizeof(float2)));
  return MINIATTN_OK;
}

// Forward launch shared by miniattn_fwd and miniattn_fwd_balanced (scratch == nullptr: plain).
static int fwd_common(const MiniAttnFwdParams* p, void* scratch, size_t scratch_bytes, void* stream) {
  g_err[0] = 0;
  int rc = check_fwd_params(p);
  if (rc != 0) return rc > 0 ? MINIATTN_OK : rc;
  const bool has_keys = p->Nk > 0;
  int sms = 0;
  if ((rc = check_device(&sms)) != 0) return rc;

  const CUtensorMapDataType dt =
      p->dtype == MINIATTN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap tm[4];
  if ((rc = make_map(&tm[0], p->q, 2, dt, p->D, p->Nq, p->Hq, p->B, p->q_stride, ma::kBoxCols,
                     ma::kTileM, "q")) != 0)
    return rc;
  if (has_keys) {
    if ((rc = make_map(&tm[1], p->k, 2, dt, p->D, p->Nk, p->Hkv, p->B, p->k_stride, ma::kBoxCols,
                       ma::kTileN, "k")) != 0)
      return rc;
    if ((rc = make_map(&tm[2], p->v, 2, dt, p->D, p->Nk, p->Hkv, p->B, p->v_stride, ma::kBoxCols,
                       ma::kTileN, "v")) != 0)
      return rc;
  } else {
    tm[1] = tm[0];
    tm[2] = tm[0];
  }
  if (p->o == nullptr) {
    tm[3] = tm[0];  // state-only call: the kernel never stores through the output map
  } else if ((rc = make_map(&tm[3], p->o, 2, dt, p->D, p->Nq, p->Hq, p->B, p->o_stride, ma::kBoxCols,
                            ma::kTileM, "o")) != 0) {
    return rc;
  }

  ma::FwdArgs a;
  fill_args(p, &a);
  const int kd = kernel_head_dim(p->D);
  const bool carry = p->carry_in || p->carry_out;
  if (carry) {
    a.carry_tiles = p->carry_tiles > 0 ? p->carry_tiles : a.n_q_tiles;
    a.carry_tile0 = p->carry_tile0;
    const size_t rows = static_cast<size_t>(p->B) * p->Hq * a.carry_tiles * ma::kTileM;
    a.carry_o = static_cast<float*>(p->carry);
    a.carry_ml = reinterpret_cast<float2*>(static_cast<uint8_t*>(p->carry) + rows * kd * sizeof(float));
    a.carry_mode = (p->carry_in ? 1 : 0) | (p->carry_out ? 2 : 0);
  }

  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int kernel = p->kernel;
  if (kernel == MINIATTN_KERNEL_AUTO) kernel = MINIATTN_KERNEL_WS;
  cudaError_t e;
  if (kernel == MINIATTN_KERNEL_SIMPLE) {
    e = ma::launch_fwd_simple(kd, p->dtype == MINIATTN_BF16, tm, a, st);
  } else {
    // a call that carries ring state always takes the plain launch
    std::shared_ptr<const ma::FwdPlan> plan;
    if (scratch != nullptr && has_keys && !carry) plan = cached_plan(a, kd, sms);
    if (plan && plan->split) {
      if ((rc = bind_scratch(*plan, kd, scratch, scratch_bytes, &a)) != 0) return rc;
      e = ma::launch_fwd_ws_plan(kd, p->dtype == MINIATTN_BF16, false, tm, a, *plan, st);
    } else {
      e = ma::launch_fwd_ws(kd, p->dtype == MINIATTN_BF16, tm, a, sms, st);
    }
  }
  if (e != cudaSuccess)
    return fail(MINIATTN_ECUDA, "kernel launch failed: %s", cudaGetErrorString(e));
  return MINIATTN_OK;
}

int miniattn_fwd(const MiniAttnFwdParams* p, void* stream) { return fwd_common(p, nullptr, 0, stream); }

int miniattn_fwd_balanced(const MiniAttnFwdParams* p, void* scratch, size_t scratch_bytes, void* stream) {
  if (scratch == nullptr && scratch_bytes != 0) {
    g_err[0] = 0;
    return fail(MINIATTN_EINVAL, "scratch is null but scratch_bytes is %zu", scratch_bytes);
  }
  return fwd_common(p, scratch, scratch_bytes, stream);
}

// Plan of a forward launch for `sm_count` SMs (<= 0: the current device's).  Host arithmetic only.
int miniattn_plan_fwd(const MiniAttnFwdParams* p, int sm_count, MiniAttnPlanInfo* info,
                      MiniAttnPlanPiece* pieces, int32_t cap) {
  g_err[0] = 0;
  if (info == nullptr) return fail(MINIATTN_EINVAL, "info is null");
  memset(info, 0, sizeof(*info));
  if (p == nullptr) return fail(MINIATTN_EINVAL, "params is null");
  if (p->D != 64 && p->D != 96 && p->D != 128)
    return fail(MINIATTN_EUNSUPPORTED, "head dim %d not supported (64, 96 or 128)", p->D);
  if (p->B < 0 || p->Hq < 0 || p->Nq < 0 || p->Nk < 0) return fail(MINIATTN_EINVAL, "negative size");
  if (p->Hq > 65535 || p->B > 65535)
    return fail(MINIATTN_EUNSUPPORTED, "B and Hq must not exceed 65535");
  int sms = sm_count;
  if (sms <= 0) {
    int rc;
    if ((rc = check_device(&sms)) != 0) return rc;
  }
  ma::FwdArgs a;
  fill_args(p, &a);
  const long long n_items = static_cast<long long>((a.n_q_tiles + 1) / 2) * p->Hq * p->B;
  info->sm_count = sms;
  info->n_ctas = n_items;
  info->head_group = a.bh_group;
  if (p->B == 0 || p->Hq == 0 || p->Nq == 0 || p->Nk == 0 ||
      (p->kernel != MINIATTN_KERNEL_AUTO && p->kernel != MINIATTN_KERNEL_WS) || p->carry_in || p->carry_out)
    return MINIATTN_OK;
  const int kd = kernel_head_dim(p->D);
  std::shared_ptr<const ma::FwdPlan> plan = cached_plan(a, kd, sms);
  info->est_plain = plan->est_plain;
  info->est_balanced = plan->est_balanced;
  if (!plan->split) return MINIATTN_OK;
  info->split = 1;
  info->n_whole = plan->n_whole;
  info->n_pieces = plan->n_table;
  info->n_ctas = plan->n_whole + plan->n_table;
  info->n_cut_items = plan->n_cut_items;
  info->n_slots = plan->n_slots;
  info->scratch_bytes = static_cast<int64_t>(scratch_bytes_of(*plan, kd));
  if (pieces != nullptr)
    for (int k = 0; k < plan->n_table && k < cap; ++k) {
      const ma::PlanEntry& e = plan->table.e[k];
      pieces[k].item = static_cast<int32_t>(e.item);
      pieces[k].t0 = e.t0;
      pieces[k].t1 = e.t1;
      pieces[k].part = e.part;
      pieces[k].nparts = e.nparts;
      pieces[k].slot = e.nparts > 1 ? e.slot0 + e.part : -1;
    }
  return MINIATTN_OK;
}

int64_t miniattn_fwd_carry_bytes(const MiniAttnFwdParams* p) {
  g_err[0] = 0;
  if (p == nullptr) return fail(MINIATTN_EINVAL, "params is null");
  if (p->D != 64 && p->D != 96 && p->D != 128)
    return fail(MINIATTN_EUNSUPPORTED, "head dim %d not supported (64, 96 or 128)", p->D);
  if (p->B < 0 || p->Hq < 0 || p->Nq < 0) return fail(MINIATTN_EINVAL, "negative size");
  const int64_t tiles = static_cast<int64_t>(p->B) * p->Hq * ((p->Nq + ma::kTileM - 1) / ma::kTileM);
  return tiles * ma::kTileM * (kernel_head_dim(p->D) * 4 + 8);
}

int64_t miniattn_fwd_balanced_scratch_bytes(const MiniAttnFwdParams* p) {
  MiniAttnPlanInfo info;
  const int rc = miniattn_plan_fwd(p, 0, &info, nullptr, 0);
  return rc != 0 ? rc : info.scratch_bytes;
}

static int check_int8_params(const MiniAttnInt8Params* p, bool need_v) {
  if (p == nullptr) return fail(MINIATTN_EINVAL, "params is null");
  MiniAttnFwdParams f = p->fwd;
  if (!need_v) {  // the pre-pass reads q and k only
    f.v = f.k;
    for (int i = 0; i < 3; ++i) f.v_stride[i] = f.k_stride[i];
    if (f.o == nullptr) {
      f.o = const_cast<void*>(f.q);
      for (int i = 0; i < 3; ++i) f.o_stride[i] = f.q_stride[i];
    }
  }
  int rc = check_fwd_params(&f);
  if (rc != 0) return rc;
  if (p->fwd.D == 96) return fail(MINIATTN_EUNSUPPORTED, "the INT8-QK variant takes head dim 64 or 128");
  if (p->fwd.carry_in || p->fwd.carry_out)
    return fail(MINIATTN_EUNSUPPORTED, "the INT8-QK variant does not carry ring state");
  if (p->fwd.Nk == 0) return fail(MINIATTN_EINVAL, "the INT8-QK variant needs at least one key");
  if (!p->q8 || !p->k8 || !p->q_scale || !p->k_scale)
    return fail(MINIATTN_EINVAL, "q8, k8, q_scale and k_scale must not be null");
  if (reinterpret_cast<uintptr_t>(p->q8) % 16 || reinterpret_cast<uintptr_t>(p->k8) % 16)
    return fail(MINIATTN_EINVAL, "q8 and k8 must be 16-byte aligned");
  return MINIATTN_OK;
}

int miniattn_quant_qk_int8(const MiniAttnInt8Params* p, void* stream) {
  g_err[0] = 0;
  int rc = check_int8_params(p, false);
  if (rc != 0) return rc > 0 ? MINIATTN_OK : rc;
  if (!p->k_partial) return fail(MINIATTN_EINVAL, "k_partial scratch must not be null");
  int sms = 0;
  if ((rc = check_device(&sms)) != 0) return rc;
  const MiniAttnFwdParams& f = p->fwd;
  const float scale = f.softmax_scale > 0.f ? f.softmax_scale : 1.0f / sqrtf((float)f.D);
  const long long qs[3] = {f.q_stride[0], f.q_stride[1], f.q_stride[2]};
  const long long ks[3] = {f.k_stride[0], f.k_stride[1], f.k_stride[2]};
  cudaError_t e = ma::launch_quant_qk(f.D, f.dtype == MINIATTN_BF16, f.q, qs, f.k, ks, f.B, f.Hq, f.Hkv,
                                      f.Nq, f.Nk, scale * 1.4426950408889634f, p->q8, p->k8, p->q_scale,
                                      p->k_scale, p->k_partial, p->k_mean,
                                      reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess)
    return fail(MINIATTN_ECUDA, "kernel launch failed: %s", cudaGetErrorString(e));
  return MINIATTN_OK;
}

int miniattn_quant_qk_int8_static(const MiniAttnInt8Params* p, void* stream) {
  g_err[0] = 0;
  int rc = check_int8_params(p, false);
  if (rc != 0) return rc > 0 ? MINIATTN_OK : rc;
  int sms = 0;
  if ((rc = check_device(&sms)) != 0) return rc;
  const MiniAttnFwdParams& f = p->fwd;
  const long long need = (long long)f.B * f.Hkv * ((f.Nk + 1023) / 1024) * f.D;
  if (need > ma::static_colsum_capacity())
    return fail(MINIATTN_EUNSUPPORTED,
                "B*Hkv*ceil(Nk/1024)*D = %lld floats of column-sum scratch exceed the built-in %lld; "
                "use miniattn_quant_qk_int8 with a caller-provided k_partial buffer",
                need, ma::static_colsum_capacity());
  const float scale = f.softmax_scale > 0.f ? f.softmax_scale : 1.0f / sqrtf((float)f.D);
  const long long qs[3] = {f.q_stride[0], f.q_stride[1], f.q_stride[2]};
  const long long ks[3] = {f.k_stride[0], f.k_stride[1], f.k_stride[2]};
  cudaError_t e = ma::launch_quant_qk_static(f.D, f.dtype == MINIATTN_BF16, f.q, qs, f.k, ks, f.B, f.Hq,
                                             f.Hkv, f.Nq, f.Nk, scale * 1.4426950408889634f, p->q8, p->k8,
                                             p->q_scale, p->k_scale, p->k_mean,
                                             reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess)
    return fail(MINIATTN_ECUDA, "pre-pass set-up or launch failed: %s", cudaGetErrorString(e));
  return MINIATTN_OK;
}

static int int8_common(const MiniAttnInt8Params* p, void* scratch, size_t scratch_bytes, void* stream) {
  g_err[0] = 0;
  int rc = check_int8_params(p, true);
  if (rc != 0) return rc > 0 ? MINIATTN_OK : rc;
  int sms = 0;
  if ((rc = check_device(&sms)) != 0) return rc;
  const MiniAttnFwdParams& f = p->fwd;
  const CUtensorMapDataType dt =
      f.dtype == MINIATTN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  // int8 rows are D bytes wide: one box per tile, 64-byte swizzle at D=64, 128-byte at D=128
  const CUtensorMapSwizzle sw8 = f.D == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  const int64_t q8s[3] = {(int64_t)f.Hq * f.Nq * f.D, (int64_t)f.Nq * f.D, f.D};
  const int64_t k8s[3] = {(int64_t)f.Hkv * f.Nk * f.D, (int64_t)f.Nk * f.D, f.D};
  CUtensorMap tm[4];
  if ((rc = make_map(&tm[0], p->q8, 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, f.D, f.Nq, f.Hq, f.B, q8s, f.D,
                     ma::kTileM, "q8", sw8)) != 0)
    return rc;
  if ((rc = make_map(&tm[1], p->k8, 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, f.D, f.Nk, f.Hkv, f.B, k8s, f.D,
                     ma::kTileN, "k8", sw8)) != 0)
    return rc;
  if ((rc = make_map(&tm[2], f.v, 2, dt, f.D, f.Nk, f.Hkv, f.B, f.v_stride, ma::kBoxCols, ma::kTileN,
                     "v")) != 0)
    return rc;
  if ((rc = make_map(&tm[3], f.o, 2, dt, f.D, f.Nq, f.Hq, f.B, f.o_stride, ma::kBoxCols, ma::kTileM,
                     "o")) != 0)
    return rc;
  ma::FwdArgs a;
  fill_args(&f, &a);
  a.sq = p->q_scale;
  a.sk = p->k_scale;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e;
  std::shared_ptr<const ma::FwdPlan> plan;
  if (scratch != nullptr) plan = cached_plan(a, f.D, sms);
  if (plan && plan->split) {
    if ((rc = bind_scratch(*plan, f.D, scratch, scratch_bytes, &a)) != 0) return rc;
    e = ma::launch_fwd_ws_plan(f.D, f.dtype == MINIATTN_BF16, true, tm, a, *plan, st);
  } else {
    e = ma::launch_fwd_ws_int8qk(f.D, f.dtype == MINIATTN_BF16, tm, a, sms, st);
  }
  if (e != cudaSuccess)
    return fail(MINIATTN_ECUDA, "kernel launch failed: %s", cudaGetErrorString(e));
  return MINIATTN_OK;
}

int miniattn_fwd_int8qk(const MiniAttnInt8Params* p, void* stream) { return int8_common(p, nullptr, 0, stream); }

int miniattn_fwd_int8qk_balanced(const MiniAttnInt8Params* p, void* scratch, size_t scratch_bytes, void* stream) {
  if (scratch == nullptr && scratch_bytes != 0) {
    g_err[0] = 0;
    return fail(MINIATTN_EINVAL, "scratch is null but scratch_bytes is %zu", scratch_bytes);
  }
  return int8_common(p, scratch, scratch_bytes, stream);
}

int miniattn_merge_partials(const MiniAttnMergeParams* p, void* stream) {
  g_err[0] = 0;
  if (p == nullptr) return fail(MINIATTN_EINVAL, "params is null");
  if (p->rows < 0) return fail(MINIATTN_EINVAL, "negative row count");
  if (p->D != 64 && p->D != 128)
    return fail(MINIATTN_EUNSUPPORTED, "head dim %d not supported (64 or 128)", p->D);
  if (p->dtype != MINIATTN_FP16 && p->dtype != MINIATTN_BF16)
    return fail(MINIATTN_EUNSUPPORTED, "dtype must be fp16 (0) or bf16 (1), got %d", p->dtype);
  if (p->init != 0 && p->init != 1) return fail(MINIATTN_EINVAL, "init must be 0 or 1");
  if (p->rows == 0) return MINIATTN_OK;
  if (!p->acc_o || !p->acc_lse || !p->part_o || !p->part_lse)
    return fail(MINIATTN_EINVAL, "acc_o, acc_lse, part_o and part_lse must not be null");
  if (reinterpret_cast<uintptr_t>(p->acc_o) % 16 || reinterpret_cast<uintptr_t>(p->part_o) % 16 ||
      (p->out && reinterpret_cast<uintptr_t>(p->out) % 16))
    return fail(MINIATTN_EINVAL, "acc_o, part_o and out must be 16-byte aligned");
  int sms = 0, rc;
  if ((rc = check_device(&sms)) != 0) return rc;
  long long rows_per_slab = p->rows, slab_stride = p->rows * p->D;
  if (p->out_rows_per_slab > 0) {
    if (p->rows % p->out_rows_per_slab != 0)
      return fail(MINIATTN_EINVAL, "rows must be a multiple of out_rows_per_slab");
    if (p->out_slab_stride < p->out_rows_per_slab * p->D || p->out_slab_stride % 8 != 0)
      return fail(MINIATTN_EINVAL, "out_slab_stride must be a multiple of 8 elements and cover a slab");
    rows_per_slab = p->out_rows_per_slab;
    slab_stride = p->out_slab_stride;
  }
  cudaError_t e = ma::launch_merge_partials(p->acc_o, p->acc_lse, p->part_o, p->part_lse, p->out,
                                            p->rows, p->D, p->dtype == MINIATTN_BF16, p->init,
                                            rows_per_slab, slab_stride, sms,
                                            reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess)
    return fail(MINIATTN_ECUDA, "kernel launch failed: %s", cudaGetErrorString(e));
  return MINIATTN_OK;
}

int miniattn_check_status(int32_t status_word) {
  g_err[0] = 0;
  if (status_word == 0) return MINIATTN_OK;
  static const char* const names[] = {"K/V or Q tile load", "S = QK^T", "O += PV", "P hand-off", "ring slot release",
                                      "correction hand-off", "partial of another CTA of a cut item"};
  char list[256] = "";
  for (int bit = 0; bit < 7; ++bit)
    if (status_word & (1 << bit)) {
      if (list[0]) strncat(list, ", ", sizeof(list) - strlen(list) - 1);
      strncat(list, names[bit], sizeof(list) - strlen(list) - 1);
    }
  if (status_word & (1 << 30)) {
    if (list[0]) strncat(list, ", ", sizeof(list) - strlen(list) - 1);
    strncat(list, "self-test wait", sizeof(list) - strlen(list) - 1);
  }
  return fail(MINIATTN_EDEVICE_WAIT, "bounded device waits ran out (status word 0x%x): %s", status_word, list);
}

int miniattn_selftest_wait(int32_t* status, uint64_t limit_ns, void* stream) {
  g_err[0] = 0;
  if (status == nullptr) return fail(MINIATTN_EINVAL, "status is null");
  if (limit_ns == 0 || limit_ns > 2000000000ull)
    return fail(MINIATTN_EINVAL, "limit_ns must be in (0, 2e9]");
  cudaError_t e = ma::launch_wait_selftest(status, limit_ns, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess)
    return fail(MINIATTN_ECUDA, "kernel launch failed: %s", cudaGetErrorString(e));
  return MINIATTN_OK;
}

}  // extern "C"
