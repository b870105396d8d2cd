/*
 * miniattn.h — C ABI of the B200 (sm_100a) FlashAttention-2 forward operator.
 *
 * One shared library (libminiattn.so), plain pointers and sizes, no torch types.
 * Every entry point returns 0 on success or a negative MINIATTN_E* code; the
 * text of the last failure on the calling thread is returned by
 * miniattn_last_error_string().  Nothing here throws, traps or blocks on the
 * device: kernels are launched asynchronously on the caller's stream.
 *
 * Reference interfaces this replaces (paths inside ShlokVFX/Mini-Attention):
 *   - ext.forward(kernel_cfg, q, k, v, o, benchmark) -> (Tensor, ms)
 *       kernels/flash_attn/cuda/sm_120/kernel/flash_attention.cu:37-40,134-138
 *   - ForwardKernelArgs (pointer + stride block handed to the device kernel)
 *       kernels/flash_attn/cuda/sm_120/kernel/include/flash_attention.cuh:16-34
 *   - forward(q, k, v) operator wrapper
 *       kernels/flash_attn/cuda/sm86/inline/fp16_k1_sm86.py:265-269
 */
#ifndef MINIATTN_H_
#define MINIATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MINIATTN_OK             0
#define MINIATTN_EINVAL        -1   /* bad argument (null pointer, stride, size)          */
#define MINIATTN_EUNSUPPORTED  -2   /* shape / dtype / device not supported               */
#define MINIATTN_ECUDA         -3   /* CUDA runtime or driver call failed                 */
#define MINIATTN_EDEVICE_WAIT  -4   /* a bounded device-side wait ran out (status word)   */

#define MINIATTN_FP16 0
#define MINIATTN_BF16 1

/* kernel selector for MiniAttnFwdParams.kernel */
#define MINIATTN_KERNEL_AUTO   0
#define MINIATTN_KERNEL_SIMPLE 1    /* one 128-row Q tile per CTA, roles not specialised   */
#define MINIATTN_KERNEL_WS     2    /* warp-specialised, two ping-ponged Q tiles per CTA   */

/*
 * Forward attention O = softmax(Q K^T * scale [+ causal mask]) V.
 *
 * Replaces ForwardKernelArgs + flash_attention_forward of the reference
 * (flash_attention.cuh:16-34, flash_attention.cu:37-132) and widens it:
 * per-tensor strides (so both the reference's (B,N,H,D) layout and (B,H,N,D)
 * work without a copy), GQA/MQA head broadcast (Hkv divides Hq; KV head g
 * serves query heads g*G .. g*G+G-1, as kernels/standard/pytorch/gqa.py:38-39),
 * causal masking (key j visible to query i iff k_pos0+j <= q_pos0+i, as
 * kernels/flash_attn/triton/fp16_flash_attn_sm86.py:55-58,74-75), optional
 * log-sum-exp output.
 *
 * Strides are in ELEMENTS for the logical dims (batch, head, token); the head
 * dim is contiguous (stride 1).  Every stride must be a multiple of 8 elements
 * and every base pointer 16-byte aligned (TMA tensor-map rules).
 *
 * Head dim D: 64, 96 or 128 (the reference instantiates 128 only,
 * flash_attention.cu:77-80).  D = 96 runs on the D = 128 kernels with the
 * columns 96..127 of every tile zero-filled / clipped by the tensor maps.
 *
 * Carried state (ring / context-parallel steps; no reference counterpart, the
 * arithmetic is the split-KV merge of
 * kernels/standard/pytorch/benchmark_mla_decode_torch.py:257-266 kept
 * un-normalised): a sequence of calls over the SAME q and successive key blocks
 * can hand the rows' running (maximum, sum, un-normalised O) from call to call
 * in `carry`, a device buffer of miniattn_fwd_carry_bytes(p) bytes, 256-byte
 * aligned, whose layout is private to the library.  First call: carry_in = 0,
 * carry_out = 1; middle calls: both 1; last call: carry_in = 1, carry_out = 0 —
 * only that one writes o (and lse).  While carry_out = 1 nothing is written to
 * o, which may then be NULL.  Nothing is rounded to 16 bit between the calls.
 * Calls with carried state always take the plain launch.  A state sized for a
 * longer q (miniattn_fwd_carry_bytes of that q) also serves calls on a row
 * range of it that starts on a multiple of 128 rows: carry_tile0, carry_tiles.
 */
typedef struct MiniAttnFwdParams {
  const void* q;          /* [B, Hq,  Nq, D] logical, device memory                */
  const void* k;          /* [B, Hkv, Nk, D]                                       */
  const void* v;          /* [B, Hkv, Nk, D]                                       */
  void*       o;          /* [B, Hq,  Nq, D], same dtype as q                      */
  float*      lse;        /* optional [B, Hq, Nq] fp32 contiguous: ln(sum exp)     */
  int32_t*    status;     /* optional device word; kernels OR error bits into it   */
  int64_t q_stride[3];    /* (batch, head, token) strides of q in elements         */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  int64_t q_pos0;         /* global position of q token 0 (causal test)            */
  int64_t k_pos0;         /* global position of k token 0                          */
  int32_t B, Hq, Hkv, Nq, Nk, D;
  int32_t dtype;          /* MINIATTN_FP16 | MINIATTN_BF16                         */
  int32_t causal;         /* 0 | 1                                                 */
  float   softmax_scale;  /* <= 0 selects 1/sqrt(D) (the reference's fixed scale,  */
                          /* forward_kernel.cuh:103-105)                           */
  int32_t kernel;         /* MINIATTN_KERNEL_*                                     */
  void*   carry;          /* running state of the rows between ring steps, or NULL */
  int32_t carry_in;       /* 1: fold the state in `carry` into this call's result  */
  int32_t carry_out;      /* 1: store the new state in `carry`, write no output    */
  int32_t carry_tile0;    /* the state may cover more query rows than this call:   */
  int32_t carry_tiles;    /* it then holds carry_tiles 128-row tiles per (batch,   */
                          /* head) and this call's first row is tile carry_tile0   */
                          /* of them (Nq of the earlier rows a multiple of 128).   */
                          /* carry_tiles = 0: the state covers exactly this q.     */
} MiniAttnFwdParams;

/* Launch the forward kernel on `stream` (a cudaStream_t; NULL = default stream). */
int miniattn_fwd(const MiniAttnFwdParams* p, void* stream);

/* Bytes of the `carry` buffer for the q of `p` (B, Hq, Nq, D are read); negative MINIATTN_E* on error. */
int64_t miniattn_fwd_carry_bytes(const MiniAttnFwdParams* p);

/*
 * Balanced forward launch (no counterpart in the reference, which launches one CTA per (batch,
 * head, Q block) and leaves the balance to the hardware, flash_attention.cu:100-123).
 *
 * The kernel runs one CTA per SM, so a launch whose work items do not fill a whole number of
 * rounds leaves SMs idle in the last one (256 items on 148 SMs: 2 rounds for 1.73 rounds of
 * work).  This entry point plans the launch on the host: the key range of some items is cut into
 * pieces that separate CTAs work on; the CTAs of a cut item count themselves in on an arrival
 * counter, all but the last to arrive leave un-normalised partial results in `scratch`, and the
 * last one folds them into its own and writes the output.  The only wait between CTAs is the last
 * arriver's for partials that CTAs already running are in the middle of writing (bounded like
 * every device wait; bit 6 of the status word if it ever runs out).  When the plan predicts no
 * gain (many rounds, or too little work per item) the launch is the plain one and scratch is not
 * touched.  Results equal miniattn_fwd's up to fp32 summation order.
 *
 * scratch: device memory, 256-byte aligned, at least miniattn_fwd_balanced_scratch_bytes(p)
 * bytes.  Its first 16384 bytes (the arrival counters) must be zero before the first launch that
 * uses it; every launch leaves them zero again, unless a bounded device wait ran out (status
 * word != 0) — clear them before the next launch in that case.  Launches that may overlap on
 * the GPU need separate scratch buffers.  scratch == NULL selects the plain launch.
 */
int miniattn_fwd_balanced(const MiniAttnFwdParams* p, void* scratch, size_t scratch_bytes, void* stream);

/* Bytes of scratch the balanced launch of `p` needs on the current device (0: it would run the
 * plain launch); a negative MINIATTN_E* code on error. */
int64_t miniattn_fwd_balanced_scratch_bytes(const MiniAttnFwdParams* p);

/* The plan itself, for inspection and tests: host arithmetic only, no device call when
 * sm_count > 0 (sm_count <= 0 asks the current device).  Pointers in `p` are not read. */
typedef struct MiniAttnPlanInfo {
  int32_t split;         /* 1: some items are cut; 0: plain launch                              */
  int32_t sm_count;
  int64_t n_ctas;        /* CTAs of the launch                                                  */
  int32_t n_whole;       /* CTAs [0, n_whole) take items [0, n_whole) whole                     */
  int32_t n_pieces;      /* CTAs after them, described by `pieces`, longest first               */
  int32_t n_cut_items;   /* items covered by more than one CTA                                  */
  int32_t n_slots;       /* partial-result slots in scratch                                     */
  int64_t scratch_bytes;
  float est_plain;       /* predicted makespans in K/V-tile steps (128 keys) of one CTA         */
  float est_balanced;
  int32_t head_group;    /* items walk the (batch, head) indices in groups of this many; B*Hq = all at once */
} MiniAttnPlanInfo;

typedef struct MiniAttnPlanPiece {
  int32_t item;          /* index in launch order.  With G = head_group and P Q-tile pairs per head:  */
                         /* group item/(P*G) of G consecutive (batch, head) indices; inside it pair   */
                         /* P-1 - (item%(P*G))/G (latest rows first) and head (item%(P*G))%G          */
  int32_t t0, t1;        /* K/V tiles [t0, t1) of the item                                      */
  int32_t part, nparts;  /* nparts == 1: the whole item                                         */
  int32_t slot;          /* partial slot of a piece of a cut item, -1 otherwise                 */
} MiniAttnPlanPiece;

int miniattn_plan_fwd(const MiniAttnFwdParams* p, int sm_count, MiniAttnPlanInfo* info,
                      MiniAttnPlanPiece* pieces, int32_t cap);

/*
 * INT8-QK variant (SageAttention-style; the reference holds no code for it, only its task
 * configuration states the recipe): K is smoothed by subtracting its per-channel mean over
 * tokens, Q and the smoothed K are quantised to int8 with one symmetric fp32 scale per block of
 * 128 tokens, S = Q8 K8^T runs on tcgen05 kind::i8 with int32 accumulation and is de-quantised
 * inside the softmax; P V stays 16 bit with fp32 accumulation.
 *
 * `fwd` carries q, k, v, o, sizes, strides, dtype, causal and softmax_scale exactly as for
 * miniattn_fwd (lse and status are honoured too; q_pos0 / k_pos0 shift the causal diagonal).
 * The remaining members are caller-allocated device buffers:
 *   q8       [B, Hq,  Nq, D] int8, contiguous         k8      [B, Hkv, Nk, D] int8, contiguous
 *   q_scale  [B, Hq,  ceil(Nq/128)] fp32 (softmax_scale*log2(e) folded in)
 *   k_scale  [B, Hkv, ceil(Nk/128)] fp32
 *   k_partial  scratch, B*Hkv*ceil(Nk/1024)*D floats (column sums of K, pre-pass only)
 *   k_mean   optional [B, Hkv, D] fp32 output of the pre-pass
 * miniattn_quant_qk_int8 runs the pre-pass (fills q8, k8, q_scale, k_scale);
 * miniattn_fwd_int8qk runs the attention kernel on buffers the pre-pass filled.
 */
typedef struct MiniAttnInt8Params {
  MiniAttnFwdParams fwd;
  int8_t* q8;
  int8_t* k8;
  float*  q_scale;
  float*  k_scale;
  float*  k_partial;
  float*  k_mean;
} MiniAttnInt8Params;

int miniattn_quant_qk_int8(const MiniAttnInt8Params* p, void* stream);
int miniattn_fwd_int8qk(const MiniAttnInt8Params* p, void* stream);

/* The INT8-QK attention kernel through the balanced launch: same scratch contract and the same
 * plan as miniattn_fwd_balanced (size it with miniattn_fwd_balanced_scratch_bytes(&p->fwd)). */
int miniattn_fwd_int8qk_balanced(const MiniAttnInt8Params* p, void* scratch, size_t scratch_bytes, void* stream);

/*
 * Allocation-free form of the INT8 pre-pass.  It has no counterpart in the reference.
 *
 * Who needs it: hosts that give this library no way to get device memory of its own — a serving
 * runtime that reserved the whole GPU for its KV cache at start-up, or a plugin slot whose
 * contract forbids cudaMalloc because an allocation synchronises the device and can fail long
 * after start-up.  Such a caller owns q, k and the outputs (q8, k8, q_scale, k_scale, optional
 * k_mean) but has nowhere to put the pre-pass's internal scratch, the per-1024-token column sums
 * of K.  This entry point keeps that scratch in a fixed array inside the library instead:
 * p->k_partial is ignored (it may be NULL) and neither this call nor anything it runs calls
 * cudaMalloc, cudaFree or any other allocating routine.
 *
 * Limit: B * Hkv * ceil(Nk/1024) * D <= 65536 floats (256 KB, held by every GPU that loads the
 * library until the process exits); larger problems are refused with MINIATTN_EUNSUPPORTED and a
 * message naming both numbers.  Results are identical to miniattn_quant_qk_int8.
 *
 * The first call on each device looks up the array's device address (with that device current);
 * make that first call outside any stream capture.  It is also the moment the CUDA driver loads
 * this library's device code onto that GPU (module loading is lazy by default), array included —
 * the one step on this path that takes device memory, a few MB, and that can therefore fail on a
 * GPU whose memory is already spoken for.  So make the first call on every device at start-up,
 * BEFORE the host reserves the rest of the memory; a one-tile problem is enough.  All calls on a device share the one array,
 * which keeps whatever the last call left in it: nothing in it needs clearing (every entry that is
 * read is written earlier in the same call), but two calls whose kernels overlap on the GPU —
 * different streams, no ordering between them — race on it.  Keep such calls on one stream or
 * order them with events.
 */
int miniattn_quant_qk_int8_static(const MiniAttnInt8Params* p, void* stream);

/*
 * Log-sum-exp merge of attention partials, used by the ring (context-parallel) launcher.
 * No reference counterpart on the CUDA side; the arithmetic is the split-KV merge of
 * kernels/standard/pytorch/benchmark_mla_decode_torch.py:244-272 applied to two partials:
 *   m = max(lse_acc, lse_p); wa = e^(lse_acc-m); wb = e^(lse_p-m)
 *   o_acc = (o_acc*wa + o_p*wb)/(wa+wb);  lse_acc = m + ln(wa+wb)
 * All tensors are contiguous over `rows` = B*Hq*Nq query rows of D (64 or 128) elements.
 */
typedef struct MiniAttnMergeParams {
  float*       acc_o;     /* [rows, D] fp32 running result, updated in place            */
  float*       acc_lse;   /* [rows]    fp32 running log-sum-exp, updated in place       */
  const void*  part_o;    /* [rows, D] 16-bit normalised partial of one ring step       */
  const float* part_lse;  /* [rows]    its log-sum-exp (-inf = no visible key)          */
  void*        out;       /* optional [rows, D] 16-bit: merged result, also written here */
  int64_t rows;
  int32_t D;
  int32_t dtype;          /* dtype of part_o / out: MINIATTN_FP16 | MINIATTN_BF16       */
  int32_t init;           /* 1: acc := partial (acc_o / acc_lse are not read)           */
  int64_t out_rows_per_slab; /* 0: `out` is contiguous.  > 0: `out` is a token-range view of  */
  int64_t out_slab_stride;   /* a larger tensor: consecutive groups of out_rows_per_slab rows */
                             /* (one (batch, head) each) start out_slab_stride elements apart */
} MiniAttnMergeParams;

int miniattn_merge_partials(const MiniAttnMergeParams* p, void* stream);

/*
 * Failure-detection self-test (no reference counterpart; the reference never checks
 * its launches, flash_attention.cu:123).  Launches one CTA that waits on a barrier
 * nothing signals.  The wait gives up after `limit_ns` nanoseconds (0 < limit_ns <= 2e9),
 * ORs bit 30 into *status (device memory) and the kernel returns normally.
 */
int miniattn_selftest_wait(int32_t* status, uint64_t limit_ns, void* stream);

/*
 * Turns a status word read back from the device (MiniAttnFwdParams.status, after synchronising)
 * into a return code: 0 when it is zero, MINIATTN_EDEVICE_WAIT otherwise, with the bounded waits
 * that ran out named in miniattn_last_error_string().  After such a failure the outputs of the
 * launches that shared the word are undefined, and the arrival counters of a balanced launch's
 * scratch may be non-zero: clear the word and the first 16384 bytes of that scratch before the
 * next launch.  Host arithmetic only.
 */
int miniattn_check_status(int32_t status_word);

/* Library / build identification: "miniattn-b200 <version> sm_100a". */
const char* miniattn_version(void);

/* Text of the last error recorded on the calling thread ("" if none). */
const char* miniattn_last_error_string(void);

#ifdef __cplusplus
}
#endif
#endif /* MINIATTN_H_ */
