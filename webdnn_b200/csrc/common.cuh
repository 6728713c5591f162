// Internal declarations shared by the translation units of libwebdnn_cuda.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/webdnn_cuda.h"

// A stream-ordered arena: slabs obtained with cudaMalloc, carved by best fit, coalesced on free.
// One in-order stream per context means a block may be reused as soon as it is freed: any kernel
// enqueued later runs after every kernel that touched the block before.
struct wdc_arena {
  struct Block {
    int64_t size;
    bool free;
  };
  struct Slab {
    char* base;
    int64_t size;
    std::map<int64_t, Block> blocks;  // offset -> block
  };
  std::vector<Slab> slabs;
  std::multimap<int64_t, std::pair<int, int64_t>> free_by_size;  // size -> (slab, offset)
  std::unordered_map<void*, std::pair<int, int64_t>> live;       // ptr -> (slab, offset)
  int64_t limit = 0, reserved = 0, in_use = 0, high_water = 0;
};

struct wdc_context {
  int device = 0;
  cudaStream_t stream = nullptr;
  wdc_arena arena;
  std::string last_error;
  std::mutex mu;
  int64_t n_alloc = 0, n_free = 0, n_launch = 0, h2d_bytes = 0, d2h_bytes = 0, n_tc_launch = 0;
  int sm_count = 0;
  int* status_word = nullptr;       // device word set by kernels whose bounded waits expire
  int* status_word_host = nullptr;  // pinned mirror
  void* tc_state = nullptr;         // tensor-map cache of the tcgen05 path
  // While a run is being captured into a CUDA graph, allocations come from (and return to) a private
  // arena that the finished graph keeps: replays reuse exactly the addresses the capture saw.
  wdc_arena* capture_arena = nullptr;
  std::vector<wdc_arena*> graph_arenas;   // arenas owned by finished graphs (and by failed captures)
  std::vector<struct wdc_graph*> live_graphs;   // finished graphs not yet destroyed
  int64_t split_seq = 0;                  // creation counter of the tensor-core path's cached operand splits
  // wdc_set_option
  int opt_precision = 0;                  // 0: tf32x3 (fp32-class accuracy), 1: tf32x1 (one pass, ~1e-3 relative)
  int opt_split_k = 1;                    // 1: small outputs with long reductions may be cut into K ranges
  int opt_pdl = 1;                        // 1: contraction launches use programmatic dependent launch
  int opt_nvtx = 0;                       // 1: wdc_range_push / wdc_range_pop emit NVTX ranges
  // second stream for host-to-device transfers that overlap the kernels of `stream`
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t copy_fence = nullptr;             // recorded on `stream`, waited by `copy_stream`
  cudaEvent_t free_fence = nullptr;             // recorded on `stream` at every wdc_free of the main arena (once `copy_stream` exists)
  static const int kUploadTickets = 16;
  cudaEvent_t upload_done[kUploadTickets] = {};  // recorded on `copy_stream` after each transfer
  int64_t upload_seq = 0;
  // third stream for device-to-host transfers that the host waits for while later work is already queued
  cudaStream_t d2h_stream = nullptr;
  cudaEvent_t d2h_fence = nullptr;               // recorded on `stream`, waited by `d2h_stream`
  static const int kDownloadTickets = 32;
  cudaEvent_t download_done[kDownloadTickets] = {};
  int64_t download_seq = 0;
  // optional per-launch timing of the contraction kernels
  struct ProfRec {
    cudaEvent_t start, stop;
    double flops;
  };
  bool profile = false;
  std::vector<ProfRec> prof;
};

int wdc_fail(wdc_context* ctx, int code, const char* fmt, ...);
int wdc_check_cuda(wdc_context* ctx, cudaError_t e, const char* what);
int wdc_check_launch(wdc_context* ctx, const char* kernel);

// RAII bracket around one contraction launch when profiling is on.
struct ProfScope {
  wdc_context* ctx;
  cudaEvent_t start = nullptr;
  double flops;
  ProfScope(wdc_context* c, double f) : ctx(c), flops(f) {
    if (ctx->profile) {
      cudaEventCreate(&start);
      cudaEventRecord(start, ctx->stream);
    }
  }
  ~ProfScope() {
    if (start) {
      cudaEvent_t stop;
      cudaEventCreate(&stop);
      cudaEventRecord(stop, ctx->stream);
      ctx->prof.push_back({start, stop, flops});
    }
  }
};

#define WDC_REQUIRE(ctx, cond, ...)                                  \
  do {                                                               \
    if (!(cond)) return wdc_fail((ctx), WDC_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define WDC_CUDA(ctx, call)                                   \
  do {                                                        \
    int _s = wdc_check_cuda((ctx), (call), #call);            \
    if (_s != WDC_OK) return _s;                              \
  } while (0)

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
    else prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Grid size for a grid-stride kernel: enough CTAs to fill the SMs a few times over.
static inline int grid_for(const wdc_context* ctx, int64_t work_items, int threads, int per_sm = 8) {
  int64_t need = ceil_div64(work_items, threads);
  int64_t cap = (int64_t)ctx->sm_count * per_sm;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

// tcgen05 implicit-GEMM path (conv_tc.cu).  Returns WDC_ERR_UNSUPPORTED when the shape is outside
// what the tensor-core kernel handles, in which case the caller uses the CUDA-core kernel.
int wdc_tc_conv2d(wdc_context* ctx, const wdc_conv_desc* d, const float* x, const float* w,
                  const float* scale, const float* shift, const float* residual, float* y);
int wdc_tc_gemm(wdc_context* ctx, const wdc_gemm_desc* d, const float* A, const float* B,
                const float* C, float* Y);
void wdc_tc_destroy(wdc_context* ctx);
// Looks up the device address of wdc_lstm_static's scratch array for ctx's (current) device (lstm.cu).
int wdc_lstm_static_setup(wdc_context* ctx);
// Drops every cached hi/lo split whose source (weight matrix or per-channel scale vector) overlaps the
// written range.  The range is [ptr, ptr + bytes) widened to the whole arena allocation that contains ptr:
// a write may start before a cached operand and still cover it, and a kernel never writes across two
// allocations, so "anything in the allocation that was written to" is the safe extent.  For memory that
// did not come from wdc_alloc only the given byte range counts (bytes == 0: the start address alone).
void wdc_tc_evict(wdc_context* ctx, const void* ptr, int64_t bytes);
// Every entry point that writes device memory reports its output here (the start; the length where it is
// cheap to know).
inline void wdc_note_write(wdc_context* ctx, const void* ptr, int64_t bytes = 0) {
  if (ctx && ptr && ctx->tc_state) wdc_tc_evict(ctx, ptr, bytes);
}
// Extent [*lo, *hi) of the live arena allocation (of any arena of the context) that contains p; false if none.
bool wdc_arena_extent(wdc_context* ctx, const void* p, const char** lo, const char** hi);
// A cached split with creation number `born` has been dropped: captured graphs recorded while it existed
// hold its address and must not be replayed any more (wdc_graph_launch then fails).
void wdc_graphs_note_evicted(wdc_context* ctx, int64_t born);
