// Internal declarations shared by the translation units of librt_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <string>

#include "../../include/rt_b200.h"

namespace rt {

// One row of the device-resident tensor table (80 bytes).
struct DevTensor {
  void* p;
  const void* g;
  void* m;
  void* v;
  const float* row_mean;  // centralization * mean of each gradient row, or nullptr
  int64_t numel;
  int64_t index0;         // tensor-local index of element 0 (multiple of 8)
  uint32_t tensor_id;
  uint32_t hyper_index;
  uint32_t row_len;       // elements per row of row_mean (0: one row)
  uint32_t flags;         // kVecOk
};
constexpr uint32_t kVecOk = 1u;  // all four pointers are 16-byte aligned
constexpr int kChunkShiftBit = 8;  // flags bits 8..11: a CTA covers (kPieceElems << shift) elements
constexpr int64_t kBigLaunchChunks = 65536;       // launches of at least this many 8192-element chunks ...
constexpr int64_t kLongTensorElems = 1 << 16;     // ... give tensors at least this long the longer CTAs

// Peer copies of a shared parameter region (kernel argument; n == 0 disables).
struct PushTable {
  const char* local;          // base of the region in this GPU's memory
  int64_t bytes;
  int n;                      // number of peers
  char* base[RT_MAX_PEERS];   // the region's base in each peer's memory, as mapped here
};

constexpr int kThreads = 256;
constexpr int kPieceElems = kThreads * 8;            // one iteration of a CTA: eight elements per thread
constexpr int kDefaultShift = 2;
constexpr int kChunkElems = kPieceElems << kDefaultShift;  // elements a default CTA walks through (8192)

// error plumbing -------------------------------------------------------------
int fail(int code, const std::string& msg);
int cuda_fail(cudaError_t e, const char* what);
#define RT_CUDA(call)                                   \
  do {                                                  \
    cudaError_t e__ = (call);                           \
    if (e__ != cudaSuccess) return cuda_fail(e__, #call); \
  } while (0)

struct Stats {
  std::atomic<uint64_t> kernel_launches{0}, h2d_bytes{0}, d2h_bytes{0}, h2d_copies{0}, d2h_copies{0};
};
Stats& stats();

// Peer copies of a shared gradient region (kernel argument; n == 0 disables): base[r] is the
// region in rank r's memory as mapped here, in rank order, this rank's own copy included.
struct PullTable {
  const char* local;
  int64_t bytes;
  int n;                      // number of ranks
  int self;                   // this rank's index (its copy is read from t.g directly)
  int staged;                 // set by the launcher: 0, or the number of shared-memory slots (2..4) the peers' words are staged through
  const char* base[RT_MAX_PEERS + 1];
};

struct PeerTables {
  PushTable push;
  PullTable pull;
};

// Hyper-parameter rows passed by value with a launch.
constexpr int kPackRows = 4;
struct HyperPack {
  rt_hyper rows[kPackRows];
};

inline int dtype_size(int d) { return d == RT_F32 ? 4 : 2; }
inline bool dtype_ok(int d) { return d >= RT_BF16 && d <= RT_F16; }

// Launch the fused kernel.  Either (table, chunks, hypers) describe a multi-tensor launch of
// nblocks chunks, or they are null and `one`/`one_h` describe a single tensor.
int launch_adamw(int pd, int gd, int sd, const DevTensor* table, const uint2* chunks,
                 const rt_hyper* hypers, const DevTensor& one, const rt_hyper& one_h,
                 uint64_t seed, int64_t nblocks, cudaStream_t stream, uint32_t flags,
                 const PeerTables* peers, const HyperPack* pack);
int check_launchable(int pd, int gd, int sd, uint32_t flags, const PeerTables* peers);
int cta_shift(int64_t launch_elems, int64_t tensor_elems, bool all16);
int64_t set_cta_shift(DevTensor& t, int64_t launch_elems, int pd, int gd, int sd);
int launch_adamw_debug(int pd, int gd, int sd, const DevTensor& one, const rt_hyper& one_h,
                       uint64_t seed, const rt_debug& dbg, cudaStream_t stream);
int validate_flat(const void* p, const void* g, const void* m, const void* v, int64_t n,
                  int pd, int gd, int sd, const rt_hyper* h, int64_t index0);
uint32_t vec_flag(const void* p, const void* g, const void* m, const void* v);

}  // namespace rt
