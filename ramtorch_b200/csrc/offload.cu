// Host-offloaded optimizer step: parameters and/or moments live in pinned CPU RAM and are
// streamed through the GPU chunk by chunk.
//
// The reference does this with Tensor.to(device, non_blocking=True) on ONE stream
// (ramtorch/stochastic_optimizers/adamw.py:160-170 in, :204-222 out): H2D, compute and D2H of a
// tensor run back to back and nothing overlaps.  Here three library-owned streams form a
// pipeline over a ring of device staging slots:
//
//   copy-in stream :  [wait slot free] H2D p,g,m,v(chunk k)                 -> event in_done[k]
//   compute stream :  [wait in_done[k]] fused SR-AdamW kernel, in place     -> event run_done[k]
//   copy-out stream:  [wait run_done[k]] D2H p,m,v(chunk k)                 -> event out_done[k]
//
// so that, in steady state, the host link carries chunk k+1 in and chunk k-1 out while chunk k
// is being updated.  The pipeline state (streams, events, ring position) persists across calls
// on a device, so consecutive tensors keep the link busy without a drain in between.
#include <mutex>
#include <vector>

#include "rt_internal.h"

namespace rt {

constexpr int kMaxDepth = 8;

struct Pipe {
  int device = -1;
  cudaStream_t in = nullptr, run = nullptr, out = nullptr;
  cudaEvent_t in_done[kMaxDepth] = {}, run_done[kMaxDepth] = {}, out_done[kMaxDepth] = {};
  cudaEvent_t entry = nullptr, exit_run = nullptr, exit_out = nullptr;
  uint64_t seq = 0;           // chunks issued so far; slot = seq % depth
  void* staging = nullptr;    // ring identity: a different buffer or geometry resets the ring
  int64_t slot_bytes = 0;
  int depth = 0;
};

static std::mutex g_pipe_mu;
static Pipe g_pipes[64];

static int get_pipe(int device, Pipe** out) {
  if (device < 0 || device >= 64) return fail(RT_E_DEVICE, "device index out of range");
  Pipe& p = g_pipes[device];
  if (p.device < 0) {
    RT_CUDA(cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking));
    RT_CUDA(cudaStreamCreateWithFlags(&p.run, cudaStreamNonBlocking));
    RT_CUDA(cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking));
    for (int s = 0; s < kMaxDepth; ++s) {
      RT_CUDA(cudaEventCreateWithFlags(&p.in_done[s], cudaEventDisableTiming));
      RT_CUDA(cudaEventCreateWithFlags(&p.run_done[s], cudaEventDisableTiming));
      RT_CUDA(cudaEventCreateWithFlags(&p.out_done[s], cudaEventDisableTiming));
    }
    RT_CUDA(cudaEventCreateWithFlags(&p.entry, cudaEventDisableTiming));
    RT_CUDA(cudaEventCreateWithFlags(&p.exit_run, cudaEventDisableTiming));
    RT_CUDA(cudaEventCreateWithFlags(&p.exit_out, cudaEventDisableTiming));
    p.device = device;
  }
  *out = &p;
  return 0;
}

static int64_t round256(int64_t x) { return (x + 255) & ~(int64_t)255; }

// Where does a pointer live?  Pinned (or registered) host memory streams asynchronously; plain
// pageable host memory is accepted too, but the runtime then stages every copy itself and
// the copies no longer overlap (cudaMemcpyAsync is synchronous for pageable buffers).
static int is_host_ptr(const void* ptr, bool* host) {
  cudaPointerAttributes a{};
  RT_CUDA(cudaPointerGetAttributes(&a, ptr));
  *host = (a.type == cudaMemoryTypeHost || a.type == cudaMemoryTypeUnregistered);
  return 0;
}

}  // namespace rt

using namespace rt;

extern "C" int64_t rt_offload_staging_bytes(int64_t chunk_elems, int ring_depth, int p_dtype,
                                            int g_dtype, int state_dtype, int p_on_host,
                                            int g_on_host, int m_on_host, int v_on_host) {
  if (chunk_elems <= 0 || (chunk_elems & 7) || ring_depth < 1 || ring_depth > kMaxDepth) return RT_E_CONFIG;
  if (!dtype_ok(p_dtype) || !dtype_ok(g_dtype) || !dtype_ok(state_dtype)) return RT_E_DTYPE;
  int64_t slot = 0;
  if (p_on_host) slot += round256(chunk_elems * dtype_size(p_dtype));
  if (g_on_host) slot += round256(chunk_elems * dtype_size(g_dtype));
  if (m_on_host) slot += round256(chunk_elems * dtype_size(state_dtype));
  if (v_on_host) slot += round256(chunk_elems * dtype_size(state_dtype));
  return slot * ring_depth;
}

extern "C" int rt_adamw_sr_offload(void* p, const void* g, void* m, void* v, int64_t n,
                                   int p_dtype, int g_dtype, int state_dtype,
                                   const rt_hyper* hyper, uint64_t seed, uint32_t tensor_id,
                                   const rt_offload_cfg* cfg, void* cuda_stream) {
  if (int rc = validate_flat(p, g, m, v, n, p_dtype, g_dtype, state_dtype, hyper, 0)) return rc;
  if (!cfg) return fail(RT_E_NULL, "cfg must be non-null");
  if (hyper->centralization != 0.0f && !cfg->row_mean)
    return fail(RT_E_CONFIG, "centralization != 0 needs cfg->row_mean (the row means of the whole gradient, see rt_row_means)");
  if (cfg->row_len < 0 || cfg->row_len > 0xFFFFFFFFll) return fail(RT_E_SIZE, "row_len must fit 32 bits");
  const int64_t chunk = cfg->chunk_elems > 0 ? cfg->chunk_elems : (int64_t)16 << 20;
  const int depth = cfg->ring_depth > 0 ? cfg->ring_depth : 3;
  if ((chunk & 7) || depth < 2 || depth > kMaxDepth) return fail(RT_E_CONFIG, "chunk_elems must be a multiple of 8 and ring_depth in 2..8");
  if (n == 0) return 0;

  bool hp = false, hg = false, hm = false, hv = false;
  if (int rc = is_host_ptr(p, &hp)) return rc;
  if (int rc = is_host_ptr(g, &hg)) return rc;
  if (int rc = is_host_ptr(m, &hm)) return rc;
  if (int rc = is_host_ptr(v, &hv)) return rc;
  const int64_t need = rt_offload_staging_bytes(chunk, depth, p_dtype, g_dtype, state_dtype, hp, hg, hm, hv);
  if (need > 0 && (!cfg->staging || cfg->staging_bytes < need))
    return fail(RT_E_CONFIG, "staging buffer too small: need " + std::to_string(need) + " bytes");
  if (cfg->staging && (reinterpret_cast<uintptr_t>(cfg->staging) & 255))
    return fail(RT_E_ALIGN, "staging must be 256-byte aligned");

  int device = 0;
  RT_CUDA(cudaGetDevice(&device));
  std::lock_guard<std::mutex> lock(g_pipe_mu);
  Pipe* pipe = nullptr;
  if (int rc = get_pipe(device, &pipe)) return rc;
  // The ring's geometry comes from the staging buffer, not from this tensor: slots of
  // staging_bytes / depth, so tensors of different sizes, dtypes and residency share one ring
  // and follow each other without a drain.
  const int64_t slot_bytes = cfg->staging ? (cfg->staging_bytes / depth) & ~(int64_t)255 : 0;
  if (need / depth > slot_bytes) return fail(RT_E_CONFIG, "staging buffer too small: need " + std::to_string(need) + " bytes");
  if (pipe->staging != cfg->staging || pipe->slot_bytes != slot_bytes || pipe->depth != depth) {
    // new ring geometry: let everything that used the old one finish first
    RT_CUDA(cudaStreamSynchronize(pipe->out));
    RT_CUDA(cudaStreamSynchronize(pipe->run));
    pipe->staging = cfg->staging;
    pipe->slot_bytes = slot_bytes;
    pipe->depth = depth;
    pipe->seq = 0;
  }

  cudaStream_t user = (cudaStream_t)cuda_stream;
  // the pipeline starts after whatever the caller already enqueued (e.g. the backward pass
  // that produced device-resident gradients)
  RT_CUDA(cudaEventRecord(pipe->entry, user));
  RT_CUDA(cudaStreamWaitEvent(pipe->in, pipe->entry, 0));
  RT_CUDA(cudaStreamWaitEvent(pipe->run, pipe->entry, 0));

  const int ps = dtype_size(p_dtype), gs = dtype_size(g_dtype), ss = dtype_size(state_dtype);
  for (int64_t off = 0; off < n; off += chunk) {
    const int64_t len = std::min(chunk, n - off);
    const int slot = (int)(pipe->seq % (uint64_t)depth);
    const bool reused = pipe->seq >= (uint64_t)depth;
    pipe->seq++;
    char* base = static_cast<char*>(cfg->staging) + (int64_t)slot * slot_bytes;
    char* cur = base;
    auto carve = [&](bool host, int esize) -> char* {
      if (!host) return nullptr;
      char* r = cur;
      cur += round256(chunk * esize);
      return r;
    };
    char* sp = carve(hp, ps);
    char* sg = carve(hg, gs);
    char* sm = carve(hm, ss);
    char* sv = carve(hv, ss);

    // copy-in
    if (reused) RT_CUDA(cudaStreamWaitEvent(pipe->in, pipe->out_done[slot], 0));
    auto in = [&](char* dst, const void* src, int esize) -> int {
      if (!dst) return 0;
      RT_CUDA(cudaMemcpyAsync(dst, static_cast<const char*>(src) + off * esize, len * esize,
                              cudaMemcpyHostToDevice, pipe->in));
      stats().h2d_bytes.fetch_add((uint64_t)(len * esize), std::memory_order_relaxed);
      stats().h2d_copies.fetch_add(1, std::memory_order_relaxed);
      return 0;
    };
    if (int rc = in(sg, g, gs)) return rc;
    if (int rc = in(sm, m, ss)) return rc;
    if (int rc = in(sv, v, ss)) return rc;
    if (int rc = in(sp, p, ps)) return rc;
    RT_CUDA(cudaEventRecord(pipe->in_done[slot], pipe->in));

    // compute, in place in the slot (or in the caller's device memory)
    RT_CUDA(cudaStreamWaitEvent(pipe->run, pipe->in_done[slot], 0));
    DevTensor t{};
    t.p = sp ? (void*)sp : (void*)(static_cast<char*>(p) + off * ps);
    t.g = sg ? (const void*)sg : (const void*)(static_cast<const char*>(g) + off * gs);
    t.m = sm ? (void*)sm : (void*)(static_cast<char*>(m) + off * ss);
    t.v = sv ? (void*)sv : (void*)(static_cast<char*>(v) + off * ss);
    t.numel = len;
    t.index0 = off;      // also what finds a chunk's rows in row_mean
    t.tensor_id = tensor_id;
    t.row_mean = hyper->centralization != 0.0f ? cfg->row_mean : nullptr;
    t.row_len = (uint32_t)cfg->row_len;
    t.flags = vec_flag(t.p, t.g, t.m, t.v);
    const int64_t nblocks = set_cta_shift(t, len, p_dtype, g_dtype, state_dtype);
    if (int rc = launch_adamw(p_dtype, g_dtype, state_dtype, nullptr, nullptr, nullptr, t, *hyper, seed,
                              nblocks, pipe->run, hyper->flags, nullptr, nullptr))
      return rc;
    RT_CUDA(cudaEventRecord(pipe->run_done[slot], pipe->run));

    // copy-out
    RT_CUDA(cudaStreamWaitEvent(pipe->out, pipe->run_done[slot], 0));
    auto out = [&](void* dst, const char* src, int esize) -> int {
      if (!src) return 0;
      RT_CUDA(cudaMemcpyAsync(static_cast<char*>(dst) + off * esize, src, len * esize,
                              cudaMemcpyDeviceToHost, pipe->out));
      stats().d2h_bytes.fetch_add((uint64_t)(len * esize), std::memory_order_relaxed);
      stats().d2h_copies.fetch_add(1, std::memory_order_relaxed);
      return 0;
    };
    if (int rc = out(p, sp, ps)) return rc;
    if (int rc = out(m, sm, ss)) return rc;
    if (int rc = out(v, sv, ss)) return rc;
    RT_CUDA(cudaEventRecord(pipe->out_done[slot], pipe->out));
  }

  if (cfg->defer_join) return 0;
  // the caller's stream resumes when the last kernel and the last copy-out are done
  RT_CUDA(cudaEventRecord(pipe->exit_run, pipe->run));
  RT_CUDA(cudaEventRecord(pipe->exit_out, pipe->out));
  RT_CUDA(cudaStreamWaitEvent(user, pipe->exit_run, 0));
  RT_CUDA(cudaStreamWaitEvent(user, pipe->exit_out, 0));
  return 0;
}

extern "C" int rt_offload_join(void* cuda_stream) {
  int device = 0;
  RT_CUDA(cudaGetDevice(&device));
  std::lock_guard<std::mutex> lock(g_pipe_mu);
  if (device < 0 || device >= 64 || g_pipes[device].device < 0) return 0;  // pipeline never used
  Pipe* pipe = &g_pipes[device];
  cudaStream_t user = (cudaStream_t)cuda_stream;
  RT_CUDA(cudaEventRecord(pipe->exit_run, pipe->run));
  RT_CUDA(cudaEventRecord(pipe->exit_out, pipe->out));
  RT_CUDA(cudaStreamWaitEvent(user, pipe->exit_run, 0));
  RT_CUDA(cudaStreamWaitEvent(user, pipe->exit_out, 0));
  return 0;
}

extern "C" int rt_host_register(void* ptr, int64_t bytes) {
  if (!ptr || bytes <= 0) return fail(RT_E_NULL, "ptr must be non-null and bytes positive");
  RT_CUDA(cudaHostRegister(ptr, (size_t)bytes, cudaHostRegisterPortable));
  return 0;
}

extern "C" int rt_host_unregister(void* ptr) {
  if (!ptr) return fail(RT_E_NULL, "ptr must be non-null");
  RT_CUDA(cudaHostUnregister(ptr));
  return 0;
}
