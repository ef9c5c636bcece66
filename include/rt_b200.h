/*
 * rt_b200.h — C ABI of librt_b200.so: the stochastic-rounding AdamW optimizer step of
 * RamTorch (ramtorch/stochastic_optimizers/adamw.py) as hand-written CUDA for sm_100a.
 *
 * Conventions
 *   - Every entry point returns int: 0 = ok, negative = argument error found on the host
 *     before any launch (RT_E_*), positive = a cudaError_t passed through.
 *     rt_last_error() returns a thread-local message for the last non-zero return.
 *   - All tensor memory belongs to the caller.  The library receives raw pointers, element
 *     counts, dtype codes and a cudaStream_t (passed as void*; NULL = the legacy default
 *     stream).  It keeps nothing beyond what a plan handle documents.
 *   - Calls are asynchronous with respect to the host unless stated otherwise: work is
 *     enqueued on the given stream and the caller synchronises.
 *   - There is no CPU implementation behind any entry point.
 *
 * Arithmetic contract (identical in the CUDA kernels and in the CPU checker under oracle/)
 *   g, m, v, p are widened to fp32.  With the scalars of rt_hyper:
 *     m' = fma(one_minus_beta1, g, m * beta1)                    adamw.py:190
 *     v' = fma(one_minus_beta2 * g, g, v * beta2)                adamw.py:191
 *     pw = apply_decay ? p * decay : p                           adamw.py:197-198
 *   and then, by default,
 *     den = fma(sqrt(v'), inv_bias_correction2_sqrt, eps)        adamw.py:193-195
 *     p'  = fma(neg_step_size * m', 1 / den, pw)                 adamw.py:199-200
 *   or, with rt_hyper.flags & RT_HYPER_REFERENCE_ORDER, in the reference's own operation order
 *     den = sqrt(v') / bias_correction2_sqrt + eps
 *     p'  = pw + (neg_step_size * m') / den
 *   Every operation (*, /, +, sqrt, 1/x, fma) is a single correctly rounded IEEE-754 binary32
 *   operation, so both forms are reproducible bit for bit on a CPU (sqrtf, fmaf, 1.0f / x).
 *   m' and v' do not depend on the flag.  The default form replaces a division by a multiply-add
 *   and the other by a reciprocal; it stays within 1e-6 of the reference order relative to
 *   max(|p|, |p' - p|) (4e-7 worst case observed), which is the reproducibility the reference itself has
 *   across ATen CPU builds, and it is what lets the all-bf16 kernel run at HBM speed.
 *   Write-back (adamw.py:204-222): a bf16 destination is stochastically rounded,
 *     out16 = ((bits(x) + r16) & 0xFFFF0000) >> 16                adamw.py:6-30
 *   an fp32 destination is copied, an fp16 destination is rounded to nearest-even.
 *
 * Random bits
 *   r16 comes from Philox4x32-10 (Salmon et al., SC'11) with
 *     key     = (seed & 0xFFFFFFFF, seed >> 32)
 *     counter = (i >> 3, tensor_id, step, stream)       i = element index inside its tensor
 *   stream 0 rounds the parameter, 1 exp_avg ("ema"), 2 exp_avg_sq ("ema_squared").
 *   The 4 output words hold 8 draws; element i takes draw j = i & 7:
 *     word = out[j >> 1];  r16 = (j & 1) ? word >> 16 : word & 0xFFFF.
 *   The bits depend only on (seed, step, tensor_id, i), never on launch geometry, chunking,
 *   residency (HBM or host) or the number of GPUs.
 *   The reference draws from torch.Generator seeded step+42 / +69 / +420 (adamw.py:206-218);
 *   that stream is not reproducible across devices and is replaced on purpose.
 */
#ifndef RT_B200_H
#define RT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype codes */
enum { RT_BF16 = 0, RT_F32 = 1, RT_F16 = 2 };

/* host-side argument errors */
enum {
  RT_E_NULL = -1,       /* required pointer is NULL */
  RT_E_DTYPE = -2,      /* dtype code outside RT_BF16..RT_F16 */
  RT_E_SIZE = -3,       /* negative or too large element count */
  RT_E_ALIGN = -4,      /* pointer not aligned to its element size */
  RT_E_PLAN = -5,       /* bad plan handle / plan misuse */
  RT_E_CONFIG = -6,     /* bad pipeline configuration */
  RT_E_DEVICE = -7      /* no usable CUDA device */
};

/*
 * Per-step scalars, already reduced to fp32 the way the reference reduces its Python
 * doubles when they meet fp32 tensors (adamw.py:186-200).  With t = step (after the
 * increment of adamw.py:177), ss = lr / (1 - beta1^t):
 */
typedef struct rt_hyper {
  float beta1;                  /* f32(beta1) */
  float one_minus_beta1;        /* f32(1 - beta1) */
  float beta2;                  /* f32(beta2) */
  float one_minus_beta2;        /* f32(1 - beta2) */
  float bias_correction2_sqrt;  /* f32(sqrt(1 - beta2^t)) */
  float eps;                    /* f32(eps) */
  float decay;                  /* f32(1 - ss * weight_decay) */
  float neg_step_size;          /* f32(-ss) */
  float centralization;         /* f32(c); 0 disables (adamw.py:179-184) */
  uint32_t apply_decay;         /* weight_decay != 0 (adamw.py:197) */
  uint32_t step;                /* t; also the Philox counter word 2 */
  uint32_t flags;               /* RT_HYPER_* bits; every row of one call must agree */
  float inv_bias_correction2_sqrt; /* f32(1 / bias_correction2_sqrt), the division in double */
  uint32_t reserved[3];
} rt_hyper;

/* rt_hyper.flags; bits not listed here are rejected with RT_E_CONFIG */
/* Bit 0 is retired (it selected approximate square root and reciprocal while the exact update
 * was bound by instruction issue; the exact default now runs at HBM speed). */
/* One Philox block per eight elements instead of three: the block of stream 0 also serves
 * the moments, read two lanes further per stream -- element i of stream s takes draw
 * ((i & 7) + 2*s) & 7 of the block of its group.  Each rounding still sees a uniform 16-bit
 * draw and stays unbiased, and the three roundings of any ONE element use three different
 * draws.  What is given up is independence between the rounding of p[i], ema[i-2] and
 * ema_squared[i-4] inside one group of eight: they compare one and the same 16-bit number with
 * their own thresholds, so their round-up events are nested, with correlation
 * (min(fa, fb) - fa fb) / sqrt(fa (1 - fa) fb (1 - fb)) for discarded fractions fa and fb (1 when
 * the fractions are equal; measured to that formula in the tests).  (The reference shares one stream
 * between ALL tensors of a step, adamw.py:206-218.)  Results remain bit-identical to the CPU
 * checker run with the same flag.  Only matters when the moments are bf16.  (The Python AdamW
 * sets it unless told otherwise; at this ABI nothing is set by default.) */
#define RT_HYPER_SHARED_DRAWS 2u
/* den and p' in the reference's operation order (see "Arithmetic contract"): one IEEE square
 * root and two IEEE divisions per element.  Bit-identical to the reference's vectorised CPU step
 * in all but ~1e-4 of the elements (where ATen's sqrt is itself not correctly rounded); about
 * 15 % slower than the default when every operand is bf16. */
#define RT_HYPER_REFERENCE_ORDER 4u

/* Fill an rt_hyper from the constructor-level values, in double precision, as
 * adamw.py:173-188 does.  Pure host arithmetic. */
int rt_hyper_fill(rt_hyper* out, double lr, double beta1, double beta2, double eps,
                  double weight_decay, double centralization, uint32_t step);

const char* rt_last_error(void);
/* Library / kernel identification, e.g. "rt_b200 0.1 sm_100a". */
const char* rt_version(void);

/* Optional per-call debug taps.  Any pointer may be NULL.
 *   rand_*  : injected 16-bit draws (device, one uint16 per element) used INSTEAD of Philox.
 *   f32_*   : device buffers receiving the fp32 values p', m', v' before the write-back.
 * Production calls pass NULL for the whole struct. */
typedef struct rt_debug {
  const uint16_t* rand_p;
  const uint16_t* rand_m;
  const uint16_t* rand_v;
  float* f32_p;
  float* f32_m;
  float* f32_v;
} rt_debug;

/*
 * Stochastic rounding alone: replaces copy_stochastic_(target, source, seed)
 * (adamw.py:6-30).  source: n fp32 on the device; target: n bf16 on the device.
 * rand16 != NULL injects the draws, otherwise Philox (seed, tensor_id, step, stream).
 */
int rt_sr_round_bf16(void* target_bf16, const float* source_f32, int64_t n,
                     const uint16_t* rand16, uint64_t seed, uint32_t tensor_id,
                     uint32_t step, uint32_t stream_id, void* cuda_stream);

/*
 * One fused step over ONE contiguous tensor resident in device memory: replaces the
 * body of AdamW.step for one parameter (adamw.py:160-222).  p, m, v are updated in place.
 * index0 is the tensor-local index of element 0 of the pointers given (non-zero when the
 * caller passes a slice of a larger tensor, e.g. a streamed chunk or a ZeRO shard); it must
 * be a multiple of 8.
 */
int rt_adamw_sr_flat(void* p, const void* g, void* m, void* v, int64_t n,
                     int p_dtype, int g_dtype, int state_dtype,
                     const rt_hyper* hyper, uint64_t seed, uint32_t tensor_id,
                     int64_t index0, const float* row_mean, int64_t row_len,
                     const rt_debug* debug, void* cuda_stream);

/*
 * Self-test of the kernels' square root and reciprocal.  No counterpart in the reference.
 * The default contract needs sqrt(v') and 1/den correctly rounded; the kernels build both for
 * two elements at a time from the hardware approximations and packed fused multiply-adds, and
 * fall back to the CUDA built-ins outside the range where that is exact.  This entry point
 * compares the pair routines with __fsqrt_rn / __frcp_rn on every one of the 2^32 binary32 bit
 * patterns (~10 ms) and writes four uint64 counters to counts_dev (device memory):
 *   [0] square-root mismatches for inputs in the fast range [2^-100, 2^100)      must be 0
 *   [1] reciprocal mismatches for inputs in [2^-90, 2^91] (every den the fast path can form)  must be 0
 *   [2], [3] mismatches over all bit patterns (zeros, denormals, infinities, negatives and NaNs
 *        are expected here: those inputs never reach the fast path).
 */
int rt_selftest_exact_math(uint64_t* counts_dev, void* cuda_stream);

/*
 * Gradient centralization (adamw.py:179-184): out[r] = mean over row r of g, fp32, for a
 * gradient viewed as rows x row_len (rows = size of dim 0, or 1 for tensors with fewer than two
 * dimensions, which the reference reduces as a whole).  The fused kernels subtract
 * centralization * out[(index0 + i) / row_len] from g[i] when a tensor carries row_mean and its
 * hyper row has centralization != 0 (row_len == 0: the whole tensor is one row).
 */
int rt_row_means(const void* g, int g_dtype, int64_t rows, int64_t row_len, float* out,
                 void* cuda_stream);

/*
 * Multi-tensor plan: the tensor table of an optimizer (one row per parameter that has a
 * gradient), uploaded to the device once and reused every step while the pointers stay
 * the same.  Replaces the Python loop of adamw.py:111-232 (~25 launches and up to three
 * generator constructions per tensor) by one launch per dtype combination.
 */
typedef struct rt_tensor_desc {
  void* p;
  const void* g;
  void* m;
  void* v;
  int64_t numel;
  int64_t index0;       /* tensor-local index of element 0 (multiple of 8) */
  uint32_t tensor_id;   /* Philox counter word 1 */
  uint32_t hyper_index; /* row of the hyper table passed at step time */
  uint8_t p_dtype, g_dtype, state_dtype, reserved0;
  uint32_t row_len;     /* elements per row for centralization; 0 = whole tensor is one row */
  const float* row_mean; /* device array of row means (rt_row_means) or NULL */
} rt_tensor_desc;

typedef struct rt_plan rt_plan;

/* Build a plan for `count` tensors on CUDA device `device`.  Allocates device memory for the
 * tables with cudaMalloc (freed by rt_plan_destroy).  Synchronous. */
int rt_plan_create(rt_plan** out, const rt_tensor_desc* tensors, int64_t count, int device);
int rt_plan_destroy(rt_plan* plan);
/* Replace the gradient pointers only (grads are re-allocated by autograd after
 * zero_grad(set_to_none=True)); `g` has one entry per plan tensor, in plan order. */
int rt_plan_set_grads(rt_plan* plan, const void* const* g, void* cuda_stream);
/* Number of kernel launches one rt_adamw_sr_multi call issues for this plan. */
int rt_plan_launches(const rt_plan* plan);
/* One optimizer step over every tensor of the plan.  hyper[] has hyper_count rows
 * (<= 1024); each tensor uses row hyper_index. */
int rt_adamw_sr_multi(rt_plan* plan, const rt_hyper* hyper, int hyper_count,
                      uint64_t seed, void* cuda_stream);

/*
 * ZeRO-1 fused redistribution (replaces the per-tensor dist.broadcast of zero1.py:78-91 for
 * the tensors this rank owns).  `local_base`/`bytes` describe a parameter region of this GPU
 * that every peer maps at the same layout; peer_base[k] is the same region in peer k's
 * memory as mapped into this process (CUDA IPC / VMM peer mapping).  While set, every
 * rt_adamw_sr_multi of the plan also stores each updated parameter that lies inside the
 * region into all peers' copies with plain peer stores, so the owners' values reach every
 * rank without a separate all-gather pass.  The caller still has to order the peers' reads
 * after all ranks' launches (any barrier-like collective on the same streams).
 * push == NULL or n_peers == 0 clears it.
 */
#define RT_MAX_PEERS 15
typedef struct rt_push {
  void* local_base;
  int64_t bytes;
  int n_peers;
  void* peer_base[RT_MAX_PEERS];
} rt_push;
int rt_plan_set_push(rt_plan* plan, const rt_push* push);

/*
 * ZeRO-2 fused reduction (replaces the per-tensor dist.reduce of zero2.py:27-57 for the tensors
 * this rank owns).  `local_base`/`bytes` describe a gradient region of this GPU that every
 * rank keeps at the same layout; base[r] is rank r's copy as mapped into this process, in rank
 * order, this rank's own included.  While set, every rt_adamw_sr_multi of the plan takes, for
 * each tensor whose gradient pointer lies inside the region, g = ((g_0 + g_1) + ...) + g_{n-1}
 * (fp32, rank order, plain peer loads) instead of the local gradient, so no reduce-scatter pass
 * is needed and the sum is not rounded to the gradient dtype.  The caller orders the launch
 * after every rank has finished writing its gradients, and the next writes after every rank's
 * launch (barrier-like collectives on the same streams).  pull == NULL or n_ranks == 0 clears it.
 */
typedef struct rt_pull {
  const void* local_base;
  int64_t bytes;
  int n_ranks;
  int self_rank;        /* index of this rank in base[] */
  const void* base[RT_MAX_PEERS + 1];
} rt_pull;
int rt_plan_set_pull(rt_plan* plan, const rt_pull* pull);

/*
 * Multi-tensor step for callers that must not allocate.  No counterpart in the reference.
 *
 * rt_plan_create keeps its tensor, chunk and hyper-parameter tables in memory it obtains from
 * cudaMalloc.  Some hosts of this library cannot do that: a process that has handed all of
 * its device memory to its own pool (a raw cudaMalloc then fails or fragments the pool), or
 * code running in a phase where the CUDA allocator is off limits because it synchronises
 * the device.  This entry point performs the same update as rt_plan_create +
 * rt_adamw_sr_multi but keeps the tables in a fixed array that is part of the library image
 * (about 595 KiB of device memory on every GPU that loads the library, until exit).  It
 * calls no cudaMalloc, cudaFree, cudaHostAlloc or any other allocating routine; parameters,
 * gradients and moments still come from the caller.
 *
 * Limits (larger requests are rejected with RT_E_SIZE and a message, nothing is launched):
 *   count <= RT_STATIC_MAX_TENSORS, hyper_count <= RT_STATIC_MAX_HYPER,
 *   sum over tensors of ceil(numel / 8192) <= RT_STATIC_MAX_CHUNKS (512 Mi elements when
 *   every tensor is a multiple of 8192 long).
 *
 * The first call on a device looks up the array's device address (with that device
 * current); make that first call before starting any stream capture.  That first call, and the
 * first use of each dtype combination on a device, also make the CUDA runtime load the code of
 * the kernels involved, which the driver may do with allocations of its own: a caller whose
 * allocation-free phase is strict runs one small warm-up call per combination before entering
 * it.  From then on a call allocates nothing anywhere.  All calls on a device
 * share the one array: each call overwrites the part of the tables it uses (nothing needs
 * to start at zero), so two calls whose GPU work can overlap -- different streams without an
 * ordering between them -- race on it.  Calls on one stream are ordered and safe.
 */
#define RT_STATIC_MAX_TENSORS 1024
#define RT_STATIC_MAX_CHUNKS 65536
#define RT_STATIC_MAX_HYPER 64
int rt_adamw_sr_multi_static(const rt_tensor_desc* tensors, int64_t count,
                             const rt_hyper* hyper, int hyper_count, uint64_t seed,
                             void* cuda_stream);

/*
 * Host-offloaded step (adamw.py:152-170, 204-222 when parameters and/or state live in CPU
 * RAM): streams one tensor through the GPU in chunks.  Each of p, g, m, v may be a host
 * pointer or a device pointer (pinned host memory overlaps its copies with the kernel;
 * pageable host memory works but every copy is then synchronous).  Host-resident ones are
 * staged through the ring of device buffers in `staging`, which must hold at least
 * rt_offload_staging_bytes(...) for this tensor; the slots are staging_bytes / ring_depth
 * each, so one larger buffer serves tensors of any size, dtype and residency without
 * draining the pipeline between them.  H2D, kernel and D2H run on three library-owned side
 * streams, ordered by events; the pipeline waits for work already enqueued on
 * `cuda_stream`, and `cuda_stream` is made to wait for the pipeline's completion (at the end
 * of the call, or in rt_offload_join when defer_join is set).
 */
typedef struct rt_offload_cfg {
  int64_t chunk_elems;  /* multiple of 8; 0 = default (2^24 elements) */
  int ring_depth;       /* 2..8; 0 = default 3 */
  int defer_join;       /* 0: cuda_stream waits for this call's work before the call returns;
                           1: it does not -- call rt_offload_join once after the last tensor, so
                              that consecutive tensors overlap in the pipeline */
  void* staging;        /* device memory */
  int64_t staging_bytes;
  const float* row_mean; /* gradient centralization (adamw.py:179-184): device array of the row means of
                            the WHOLE gradient (rt_row_means), required when hyper->centralization != 0,
                            else NULL */
  int64_t row_len;      /* elements per row of row_mean; 0 = the whole tensor is one row */
} rt_offload_cfg;

int64_t rt_offload_staging_bytes(int64_t chunk_elems, int ring_depth, int p_dtype,
                                 int g_dtype, int state_dtype, int p_on_host,
                                 int g_on_host, int m_on_host, int v_on_host);

int rt_adamw_sr_offload(void* p, const void* g, void* m, void* v, int64_t n,
                        int p_dtype, int g_dtype, int state_dtype,
                        const rt_hyper* hyper, uint64_t seed, uint32_t tensor_id,
                        const rt_offload_cfg* cfg, void* cuda_stream);

/* Make cuda_stream wait for everything the streaming pipeline of the current device has been
 * given so far (use with rt_offload_cfg.defer_join = 1). */
int rt_offload_join(void* cuda_stream);

/* Pin / unpin caller-owned host memory (cudaHostRegister) so the copy engines can stream it;
 * needed for shared-memory parameter storage that arrives unpinned in worker processes. */
int rt_host_register(void* ptr, int64_t bytes);
int rt_host_unregister(void* ptr);

/* Counters since load: kernels launched by this library, bytes copied H2D and D2H by the
 * offload pipeline. */
typedef struct rt_stats {
  uint64_t kernel_launches;
  uint64_t h2d_bytes;
  uint64_t d2h_bytes;
  uint64_t h2d_copies;
  uint64_t d2h_copies;
} rt_stats;
int rt_query_stats(rt_stats* out);

#ifdef __cplusplus
}
#endif
#endif /* RT_B200_H */
