// Context, stream-ordered arena, host<->device transfers and error reporting.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include <nvtx3/nvToolsExt.h>   // header-only: ranges reach a profiler only when one has injected its library

#include "common.cuh"

static std::string g_last_error;  // for failures before a context exists
static std::mutex g_mu;

int wdc_fail(wdc_context* ctx, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (ctx) {
    ctx->last_error = buf;
  } else {
    std::lock_guard<std::mutex> lk(g_mu);
    g_last_error = buf;
  }
  return code;
}

int wdc_check_cuda(wdc_context* ctx, cudaError_t e, const char* what) {
  if (e == cudaSuccess) return WDC_OK;
  int code = (e == cudaErrorMemoryAllocation) ? WDC_ERR_OOM : WDC_ERR_CUDA;
  return wdc_fail(ctx, code, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

int wdc_check_launch(wdc_context* ctx, const char* kernel) {
  ctx->n_launch++;
  return wdc_check_cuda(ctx, cudaGetLastError(), kernel);
}

extern "C" const char* wdc_last_error(wdc_context* ctx) {
  if (ctx) return ctx->last_error.c_str();
  return g_last_error.c_str();
}

extern "C" int wdc_device_count(int* count) {
  if (!count) return wdc_fail(nullptr, WDC_ERR_INVALID, "wdc_device_count: null output");
  cudaError_t e = cudaGetDeviceCount(count);
  if (e != cudaSuccess) {
    *count = 0;
    return wdc_check_cuda(nullptr, e, "cudaGetDeviceCount");
  }
  return WDC_OK;
}

__global__ void fill_u32_kernel(uint32_t* dst, uint32_t v, int64_t n);

extern "C" int wdc_create(int device, int64_t arena_limit_bytes, wdc_context** out) {
  if (!out) return wdc_fail(nullptr, WDC_ERR_INVALID, "wdc_create: null output");
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) return wdc_check_cuda(nullptr, e, "cudaGetDeviceCount");
  if (device < 0 || device >= n)
    return wdc_fail(nullptr, WDC_ERR_INVALID, "wdc_create: device %d out of range (have %d)", device, n);
  e = cudaSetDevice(device);
  if (e != cudaSuccess) return wdc_check_cuda(nullptr, e, "cudaSetDevice");
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) return wdc_check_cuda(nullptr, e, "cudaGetDeviceProperties");
  if (prop.major != 10)
    return wdc_fail(nullptr, WDC_ERR_UNSUPPORTED,
                    "wdc_create: device %d is sm_%d%d; this library carries sm_100a code only",
                    device, prop.major, prop.minor);
  wdc_context* ctx = new wdc_context();
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->arena.limit = arena_limit_bytes;
  e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaMalloc((void**)&ctx->status_word, 256);
  if (e == cudaSuccess) e = cudaMemset(ctx->status_word, 0, 256);
  if (e == cudaSuccess) e = cudaMallocHost((void**)&ctx->status_word_host, 256);
  if (e != cudaSuccess) {
    int s = wdc_check_cuda(nullptr, e, "wdc_create");
    delete ctx;
    return s;
  }
  memset(ctx->status_word_host, 0, 256);
  // wdc_lstm_static's scratch array: its address is resolved (and its module loaded, which is when the
  // driver sets the array aside) here, so that the entry point itself never reaches an allocator
  int s = wdc_lstm_static_setup(ctx);
  if (s == WDC_OK) {
    cudaFuncAttributes fa;   // this file's module too (wdc_fill_u32 is part of that entry point's sequence)
    s = wdc_check_cuda(ctx, cudaFuncGetAttributes(&fa, fill_u32_kernel), "cudaFuncGetAttributes");
  }
  if (s != WDC_OK) {
    g_last_error = ctx->last_error;
    wdc_destroy(ctx);
    return s;
  }
  *out = ctx;
  return WDC_OK;
}

extern "C" int wdc_destroy(wdc_context* ctx) {
  if (!ctx) return WDC_OK;
  DeviceGuard g(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  wdc_tc_destroy(ctx);
  for (auto& s : ctx->arena.slabs) cudaFree(s.base);
  if (ctx->capture_arena) ctx->graph_arenas.push_back(ctx->capture_arena);
  for (wdc_arena* a : ctx->graph_arenas) {
    for (auto& s : a->slabs) cudaFree(s.base);
    delete a;
  }
  cudaFree(ctx->status_word);
  cudaFreeHost(ctx->status_word_host);
  if (ctx->d2h_stream) {
    cudaStreamSynchronize(ctx->d2h_stream);
    cudaStreamDestroy(ctx->d2h_stream);
    cudaEventDestroy(ctx->d2h_fence);
    for (auto& ev : ctx->download_done)
      if (ev) cudaEventDestroy(ev);
  }
  if (ctx->copy_stream) {
    cudaStreamSynchronize(ctx->copy_stream);
    cudaStreamDestroy(ctx->copy_stream);
    cudaEventDestroy(ctx->copy_fence);
    cudaEventDestroy(ctx->free_fence);
    for (auto& ev : ctx->upload_done)
      if (ev) cudaEventDestroy(ev);
  }
  cudaStreamDestroy(ctx->stream);
  delete ctx;
  return WDC_OK;
}

static const int64_t kAlign = 512;
static const int64_t kSlabMin = 256ll << 20;

static void arena_erase_free(wdc_arena& a, int slab, int64_t off, int64_t size) {
  auto range = a.free_by_size.equal_range(size);
  for (auto it = range.first; it != range.second; ++it) {
    if (it->second.first == slab && it->second.second == off) {
      a.free_by_size.erase(it);
      return;
    }
  }
}

extern "C" int wdc_alloc(wdc_context* ctx, int64_t bytes, void** dptr) {
  if (!ctx || !dptr) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_alloc: null argument");
  *dptr = nullptr;
  if (bytes < 0) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_alloc: negative size %lld", (long long)bytes);
  std::lock_guard<std::mutex> lk(ctx->mu);
  wdc_arena& a = ctx->capture_arena ? *ctx->capture_arena : ctx->arena;
  int64_t need = ((bytes > 0 ? bytes : 1) + kAlign - 1) / kAlign * kAlign;
  if (a.limit > 0 && a.in_use + need > a.limit)
    return wdc_fail(ctx, WDC_ERR_OOM, "wdc_alloc: %lld bytes would exceed the arena budget of %lld (in use %lld)",
                    (long long)need, (long long)a.limit, (long long)a.in_use);
  auto it = a.free_by_size.lower_bound(need);
  if (it == a.free_by_size.end()) {
    DeviceGuard g(ctx->device);
    int64_t slab_size = need > kSlabMin ? need : kSlabMin;
    char* base = nullptr;
    cudaError_t e = cudaMalloc((void**)&base, (size_t)slab_size);
    if (e != cudaSuccess && slab_size > need) {
      cudaGetLastError();
      slab_size = need;
      e = cudaMalloc((void**)&base, (size_t)slab_size);
    }
    if (e != cudaSuccess) {
      cudaGetLastError();
      return wdc_fail(ctx, WDC_ERR_OOM, "wdc_alloc: cudaMalloc of %lld bytes failed: %s",
                      (long long)slab_size, cudaGetErrorString(e));
    }
    wdc_arena::Slab s;
    s.base = base;
    s.size = slab_size;
    s.blocks[0] = {slab_size, true};
    a.slabs.push_back(std::move(s));
    a.reserved += slab_size;
    it = a.free_by_size.insert({slab_size, {(int)a.slabs.size() - 1, 0}});
  }
  int slab = it->second.first;
  int64_t off = it->second.second, size = it->first;
  a.free_by_size.erase(it);
  auto& blocks = a.slabs[slab].blocks;
  if (size - need >= kAlign) {
    blocks[off] = {need, false};
    blocks[off + need] = {size - need, true};
    a.free_by_size.insert({size - need, {slab, off + need}});
  } else {
    need = size;
    blocks[off] = {size, false};
  }
  void* p = a.slabs[slab].base + off;
  a.live[p] = {slab, off};
  a.in_use += need;
  if (a.in_use > a.high_water) a.high_water = a.in_use;
  ctx->n_alloc++;
  *dptr = p;
  return WDC_OK;
}

bool wdc_arena_extent(wdc_context* ctx, const void* p, const char** lo, const char** hi) {
  std::lock_guard<std::mutex> lk(ctx->mu);
  const char* q = (const char*)p;
  auto search = [&](wdc_arena* a) -> bool {
    for (auto& s : a->slabs) {
      if (q < s.base || q >= s.base + s.size) continue;
      auto it = s.blocks.upper_bound((int64_t)(q - s.base));
      if (it == s.blocks.begin()) return false;
      --it;
      if (it->second.free) return false;
      *lo = s.base + it->first;
      *hi = *lo + it->second.size;
      return true;
    }
    return false;
  };
  if (search(&ctx->arena)) return true;
  if (ctx->capture_arena && search(ctx->capture_arena)) return true;
  for (wdc_arena* g : ctx->graph_arenas)
    if (search(g)) return true;
  return false;
}

extern "C" int wdc_free(wdc_context* ctx, void* dptr) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_free: null context");
  if (!dptr) return WDC_OK;
  wdc_tc_evict(ctx, dptr, 0);   // widened to the block's extent
  std::lock_guard<std::mutex> lk(ctx->mu);
  wdc_arena* owner = &ctx->arena;
  if (ctx->arena.live.find(dptr) == ctx->arena.live.end()) {
    owner = nullptr;
    if (ctx->capture_arena && ctx->capture_arena->live.count(dptr)) owner = ctx->capture_arena;
    for (wdc_arena* g : ctx->graph_arenas)
      if (!owner && g->live.count(dptr)) owner = g;
  }
  if (!owner)
    return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_free: %p is not a live allocation of this context", dptr);
  wdc_arena& a = *owner;
  auto lit = a.live.find(dptr);
  int slab = lit->second.first;
  int64_t off = lit->second.second;
  a.live.erase(lit);
  auto& blocks = a.slabs[slab].blocks;
  auto it = blocks.find(off);
  int64_t size = it->second.size;
  a.in_use -= size;
  ctx->n_free++;
  // coalesce with the next block
  auto nx = std::next(it);
  if (nx != blocks.end() && nx->second.free) {
    arena_erase_free(a, slab, nx->first, nx->second.size);
    size += nx->second.size;
    blocks.erase(nx);
  }
  // coalesce with the previous block
  if (it != blocks.begin()) {
    auto pv = std::prev(it);
    if (pv->second.free) {
      arena_erase_free(a, slab, pv->first, pv->second.size);
      size += pv->second.size;
      off = pv->first;
      blocks.erase(it);
      it = pv;
    }
  }
  it->second = {size, true};
  a.free_by_size.insert({size, {slab, off}});
  // A block of the main arena may be handed to a transfer on the copy stream next (wdc_upload_fresh_async): the
  // position of this free in the compute stream's order is what that transfer has to wait for.
  if (owner == &ctx->arena && ctx->copy_stream && !ctx->capture_arena) {
    DeviceGuard g(ctx->device);
    cudaEventRecord(ctx->free_fence, ctx->stream);
  }
  return WDC_OK;
}

extern "C" int wdc_host_alloc(wdc_context* ctx, int64_t bytes, void** hptr) {
  if (!ctx || !hptr || bytes < 0) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_host_alloc: bad argument");
  DeviceGuard g(ctx->device);
  WDC_CUDA(ctx, cudaMallocHost(hptr, (size_t)(bytes > 0 ? bytes : 1)));
  return WDC_OK;
}

extern "C" int wdc_host_free(wdc_context* ctx, void* hptr) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_host_free: null context");
  if (!hptr) return WDC_OK;
  DeviceGuard g(ctx->device);
  WDC_CUDA(ctx, cudaFreeHost(hptr));
  return WDC_OK;
}

extern "C" int wdc_upload(wdc_context* ctx, void* dst, const void* host, int64_t bytes) {
  if (!ctx || bytes < 0 || (bytes > 0 && (!dst || !host)))
    return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_upload: bad argument");
  if (bytes == 0) return WDC_OK;
  DeviceGuard g(ctx->device);
  wdc_tc_evict(ctx, dst, bytes);
  WDC_CUDA(ctx, cudaMemcpyAsync(dst, host, (size_t)bytes, cudaMemcpyHostToDevice, ctx->stream));
  ctx->h2d_bytes += bytes;
  return WDC_OK;
}

static int upload_async(wdc_context* ctx, void* dst, const void* host, int64_t bytes, int64_t* ticket, bool fresh) {
  if (!ctx || !ticket || bytes < 0 || (bytes > 0 && (!dst || !host)))
    return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_upload_async: bad argument");
  DeviceGuard g(ctx->device);
  if (!ctx->copy_stream) {
    WDC_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
    WDC_CUDA(ctx, cudaEventCreateWithFlags(&ctx->copy_fence, cudaEventDisableTiming));
    WDC_CUDA(ctx, cudaEventCreateWithFlags(&ctx->free_fence, cudaEventDisableTiming));
    for (auto& ev : ctx->upload_done) WDC_CUDA(ctx, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    // every free before this moment had no fence of its own: this one stands for them all
    WDC_CUDA(ctx, cudaEventRecord(ctx->free_fence, ctx->stream));
  }
  wdc_tc_evict(ctx, dst, bytes);
  if (fresh) {
    // dst is untouched since wdc_alloc returned it: only a previous tenant of the memory can still be in use, and
    // it was freed no later than the arena's most recent free
    WDC_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->free_fence, 0));
  } else {
    // the transfer may start only after everything already queued on `stream` (work that reads or writes dst, or a
    // previous tenant of its memory)
    WDC_CUDA(ctx, cudaEventRecord(ctx->copy_fence, ctx->stream));
    WDC_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->copy_fence, 0));
  }
  if (bytes > 0)
    WDC_CUDA(ctx, cudaMemcpyAsync(dst, host, (size_t)bytes, cudaMemcpyHostToDevice, ctx->copy_stream));
  const int64_t t = ctx->upload_seq++;
  WDC_CUDA(ctx, cudaEventRecord(ctx->upload_done[t % wdc_context::kUploadTickets], ctx->copy_stream));
  ctx->h2d_bytes += bytes;
  *ticket = t;
  return WDC_OK;
}

extern "C" int wdc_upload_async(wdc_context* ctx, void* dst, const void* host, int64_t bytes, int64_t* ticket) {
  return upload_async(ctx, dst, host, bytes, ticket, false);
}

extern "C" int wdc_upload_fresh_async(wdc_context* ctx, void* dst, const void* host, int64_t bytes, int64_t* ticket) {
  return upload_async(ctx, dst, host, bytes, ticket, true);
}

extern "C" int wdc_wait_upload(wdc_context* ctx, int64_t ticket) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_wait_upload: null context");
  if (ticket < 0 || ticket >= ctx->upload_seq)
    return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_wait_upload: unknown ticket %lld", (long long)ticket);
  // an event slot that has been reused marks a later transfer of the same in-order stream, which
  // implies this one
  DeviceGuard g(ctx->device);
  int64_t slot = ticket;
  if (ctx->upload_seq - ticket > wdc_context::kUploadTickets) slot = ctx->upload_seq - 1;
  WDC_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->upload_done[slot % wdc_context::kUploadTickets], 0));
  return WDC_OK;
}

// ---- capture of one run into a CUDA graph ------------------------------------------------------
struct wdc_graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  wdc_arena* arena = nullptr;  // owns every buffer the captured launches touch that was allocated while capturing
  // The recorded launches hold the addresses of the tensor-core path's cached operand splits (hi/lo copies of
  // the weights).  split_seq = the context's split counter when the capture ended: if a split that is that old
  // is dropped later (its weight was rewritten or freed), the graph would read freed memory, so it goes stale.
  int64_t split_seq = 0;
  bool stale = false;
};

void wdc_graphs_note_evicted(wdc_context* ctx, int64_t born) {
  for (wdc_graph* g : ctx->live_graphs)
    if (born <= g->split_seq) g->stale = true;
}

extern "C" int wdc_capture_begin(wdc_context* ctx) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_capture_begin: null context");
  if (ctx->capture_arena) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_capture_begin: a capture is already open");
  if (ctx->profile) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_capture_begin: switch per-launch profiling off first");
  DeviceGuard g(ctx->device);
  // relaxed mode: growing the private arena calls cudaMalloc, which the stricter modes refuse in this thread
  WDC_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
  ctx->capture_arena = new wdc_arena();
  return WDC_OK;
}

static void arena_release(wdc_arena* a) {
  for (auto& s : a->slabs) cudaFree(s.base);
  delete a;
}

extern "C" int wdc_capture_end(wdc_context* ctx, wdc_graph** out) {
  if (!ctx || !out) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_capture_end: null argument");
  *out = nullptr;
  if (!ctx->capture_arena) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_capture_end: no capture is open");
  DeviceGuard g(ctx->device);
  wdc_arena* arena = ctx->capture_arena;
  ctx->capture_arena = nullptr;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
  // blocks of the main arena that were freed while the capture was open got no fence of their own (an event record
  // would have been captured): this one stands for them
  if (ctx->copy_stream) cudaEventRecord(ctx->free_fence, ctx->stream);
  cudaGraphExec_t exec = nullptr;
  if (e == cudaSuccess) e = cudaGraphInstantiate(&exec, graph, 0);
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (graph) cudaGraphDestroy(graph);
    // buffers handed out during the failed capture stay valid until their owners free them
    ctx->graph_arenas.push_back(arena);
    return wdc_fail(ctx, WDC_ERR_CUDA, "wdc_capture_end: %s", cudaGetErrorString(e));
  }
  wdc_graph* gr = new wdc_graph();
  gr->graph = graph;
  gr->exec = exec;
  gr->arena = arena;
  gr->split_seq = ctx->split_seq;
  ctx->graph_arenas.push_back(arena);
  ctx->live_graphs.push_back(gr);
  *out = gr;
  return WDC_OK;
}

extern "C" int wdc_graph_launch(wdc_context* ctx, wdc_graph* graph) {
  if (!ctx || !graph || !graph->exec) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_graph_launch: bad argument");
  if (ctx->capture_arena) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_graph_launch: a capture is open");
  if (graph->stale)
    return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_graph_launch: a weight or scale buffer the captured run uses was "
                    "rewritten or freed after the capture; destroy this graph and capture the run again");
  DeviceGuard g(ctx->device);
  WDC_CUDA(ctx, cudaGraphLaunch(graph->exec, ctx->stream));
  ctx->n_launch++;
  return WDC_OK;
}

extern "C" int wdc_graph_destroy(wdc_context* ctx, wdc_graph* graph) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_graph_destroy: null context");
  if (!graph) return WDC_OK;
  DeviceGuard g(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  for (size_t i = 0; i < ctx->live_graphs.size(); i++)
    if (ctx->live_graphs[i] == graph) ctx->live_graphs.erase(ctx->live_graphs.begin() + i--);
  if (graph->exec) cudaGraphExecDestroy(graph->exec);
  if (graph->graph) cudaGraphDestroy(graph->graph);
  if (graph->arena) {
    if (!graph->arena->live.empty())
      wdc_fail(ctx, WDC_ERR_INVALID, "wdc_graph_destroy: %zu buffers of the captured run are still allocated; they are "
               "released with the graph", graph->arena->live.size());
    for (size_t i = 0; i < ctx->graph_arenas.size(); i++)
      if (ctx->graph_arenas[i] == graph->arena) ctx->graph_arenas.erase(ctx->graph_arenas.begin() + i--);
    arena_release(graph->arena);
  }
  delete graph;
  return WDC_OK;
}

static int report_device_status(wdc_context* ctx) {
  // status_word_host is refreshed by the download/sync paths below
  if (ctx->status_word_host[0] != 0) {
    int code = ctx->status_word_host[0];
    ctx->status_word_host[0] = 0;
    cudaMemsetAsync(ctx->status_word, 0, 256, ctx->stream);
    return wdc_fail(ctx, WDC_ERR_DEVICE_WAIT, "a bounded device-side wait expired (kernel status %d)", code);
  }
  return WDC_OK;
}

extern "C" int wdc_sync(wdc_context* ctx) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_sync: null context");
  DeviceGuard g(ctx->device);
  WDC_CUDA(ctx, cudaMemcpyAsync(ctx->status_word_host, ctx->status_word, sizeof(int),
                                cudaMemcpyDeviceToHost, ctx->stream));
  WDC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return report_device_status(ctx);
}

extern "C" int wdc_download(wdc_context* ctx, void* host, const void* src, int64_t bytes) {
  if (!ctx || bytes < 0 || (bytes > 0 && (!host || !src)))
    return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_download: bad argument");
  DeviceGuard g(ctx->device);
  if (bytes > 0) {
    WDC_CUDA(ctx, cudaMemcpyAsync(host, src, (size_t)bytes, cudaMemcpyDeviceToHost, ctx->stream));
    ctx->d2h_bytes += bytes;
  }
  return wdc_sync(ctx);
}

extern "C" int wdc_download_async(wdc_context* ctx, void* host, const void* src, int64_t bytes, int64_t* ticket) {
  if (!ctx || !ticket || bytes < 0 || (bytes > 0 && (!host || !src)))
    return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_download_async: bad argument");
  DeviceGuard g(ctx->device);
  if (!ctx->d2h_stream) {
    WDC_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->d2h_stream, cudaStreamNonBlocking));
    WDC_CUDA(ctx, cudaEventCreateWithFlags(&ctx->d2h_fence, cudaEventDisableTiming));
    for (auto& ev : ctx->download_done) WDC_CUDA(ctx, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  }
  if (ctx->download_seq - wdc_context::kDownloadTickets >= 0) {
    // the event slot about to be reused belongs to a transfer issued kDownloadTickets calls ago: make sure it ran
    WDC_CUDA(ctx, cudaEventSynchronize(ctx->download_done[ctx->download_seq % wdc_context::kDownloadTickets]));
  }
  // the transfer reads what the work queued so far on the compute stream produces, and nothing queued later
  WDC_CUDA(ctx, cudaEventRecord(ctx->d2h_fence, ctx->stream));
  WDC_CUDA(ctx, cudaStreamWaitEvent(ctx->d2h_stream, ctx->d2h_fence, 0));
  if (bytes > 0)
    WDC_CUDA(ctx, cudaMemcpyAsync(host, src, (size_t)bytes, cudaMemcpyDeviceToHost, ctx->d2h_stream));
  // the device status word travels with it, so that wdc_wait_download can report an expired device wait
  WDC_CUDA(ctx, cudaMemcpyAsync(ctx->status_word_host, ctx->status_word, sizeof(int), cudaMemcpyDeviceToHost,
                                ctx->d2h_stream));
  const int64_t t = ctx->download_seq++;
  WDC_CUDA(ctx, cudaEventRecord(ctx->download_done[t % wdc_context::kDownloadTickets], ctx->d2h_stream));
  ctx->d2h_bytes += bytes;
  *ticket = t;
  return WDC_OK;
}

extern "C" int wdc_wait_download(wdc_context* ctx, int64_t ticket) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_wait_download: null context");
  if (ticket < 0 || ticket >= ctx->download_seq)
    return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_wait_download: unknown ticket %lld", (long long)ticket);
  DeviceGuard g(ctx->device);
  // a reused slot marks a later transfer of the same in-order stream, which implies this one
  int64_t slot = ticket;
  if (ctx->download_seq - ticket > wdc_context::kDownloadTickets) slot = ctx->download_seq - 1;
  WDC_CUDA(ctx, cudaEventSynchronize(ctx->download_done[slot % wdc_context::kDownloadTickets]));
  // a bounded device wait that expired before this point is reported here, like wdc_download does
  if (*(volatile int*)ctx->status_word_host != 0) return report_device_status(ctx);
  return WDC_OK;
}

extern "C" int wdc_copy(wdc_context* ctx, void* dst, const void* src, int64_t bytes) {
  if (!ctx || bytes < 0 || (bytes > 0 && (!dst || !src)))
    return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_copy: bad argument");
  if (bytes == 0) return WDC_OK;
  DeviceGuard g(ctx->device);
  wdc_tc_evict(ctx, dst, bytes);
  WDC_CUDA(ctx, cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return WDC_OK;
}

__global__ void fill_u32_kernel(uint32_t* dst, uint32_t v, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) dst[i] = v;
}

extern "C" int wdc_fill_u32(wdc_context* ctx, void* dst, uint32_t value, int64_t count) {
  if (!ctx || count < 0 || (count > 0 && !dst))
    return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_fill_u32: bad argument");
  wdc_note_write(ctx, dst, count * 4);
  if (count == 0) return WDC_OK;
  DeviceGuard g(ctx->device);
  fill_u32_kernel<<<grid_for(ctx, count, 256), 256, 0, ctx->stream>>>((uint32_t*)dst, value, count);
  return wdc_check_launch(ctx, "fill_u32_kernel");
}

extern "C" int wdc_set_option(wdc_context* ctx, const char* name, int64_t value) {
  if (!ctx || !name) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_set_option: null argument");
  const std::string n(name);
  if (n == "precision") {
    if (value != 0 && value != 1)
      return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_set_option: precision is 0 (tf32x3) or 1 (tf32x1), not %lld", (long long)value);
    ctx->opt_precision = (int)value;
  } else if (n == "split_k") {
    ctx->opt_split_k = value != 0;
  } else if (n == "pdl") {
    ctx->opt_pdl = value != 0;
  } else if (n == "nvtx") {
    ctx->opt_nvtx = value != 0;
  } else {
    return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_set_option: unknown option '%s'", name);
  }
  return WDC_OK;
}

extern "C" int wdc_range_push(wdc_context* ctx, const char* name) {
  if (!ctx || !name) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_range_push: null argument");
  if (ctx->opt_nvtx) nvtxRangePushA(name);
  return WDC_OK;
}

extern "C" int wdc_range_pop(wdc_context* ctx) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_range_pop: null context");
  if (ctx->opt_nvtx) nvtxRangePop();
  return WDC_OK;
}

extern "C" void* wdc_stream(wdc_context* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

extern "C" int wdc_stats(wdc_context* ctx, int64_t* out, int n) {
  if (!ctx || !out || n < 0) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_stats: bad argument");
  int64_t v[11] = {ctx->arena.in_use, ctx->arena.high_water, ctx->arena.reserved, ctx->n_alloc,
                   ctx->n_free,       ctx->n_launch,         ctx->h2d_bytes,      ctx->d2h_bytes,
                   ctx->n_tc_launch,  -1,                    -1};
  if (n > 9) {   // device-wide figures (every process and library on the GPU counts), asked only when wanted
    DeviceGuard g(ctx->device);
    size_t free_b = 0, total_b = 0;
    if (cudaMemGetInfo(&free_b, &total_b) == cudaSuccess) {
      v[9] = (int64_t)free_b;
      v[10] = (int64_t)total_b;
    } else {
      cudaGetLastError();
    }
  }
  for (int i = 0; i < n && i < 11; i++) out[i] = v[i];
  return WDC_OK;
}

extern "C" int wdc_reset_stats(wdc_context* ctx) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_reset_stats: null context");
  ctx->n_alloc = ctx->n_free = ctx->n_launch = ctx->h2d_bytes = ctx->d2h_bytes = ctx->n_tc_launch = 0;
  ctx->arena.high_water = ctx->arena.in_use;
  return WDC_OK;
}

extern "C" int wdc_profile_enable(wdc_context* ctx, int on) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_profile_enable: null context");
  ctx->profile = on != 0;
  return WDC_OK;
}

extern "C" int wdc_profile_read(wdc_context* ctx, int family, double* ms, int64_t* launches, double* flops) {
  if (!ctx || !ms || !launches || !flops || family != 0)
    return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_profile_read: bad argument");
  DeviceGuard g(ctx->device);
  WDC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  double total = 0, fl = 0;
  for (auto& r : ctx->prof) {
    float t = 0;
    cudaEventElapsedTime(&t, r.start, r.stop);
    total += t;
    fl += r.flops;
    cudaEventDestroy(r.start);
    cudaEventDestroy(r.stop);
  }
  *ms = total;
  *launches = (int64_t)ctx->prof.size();
  *flops = fl;
  ctx->prof.clear();
  return WDC_OK;
}

extern "C" int wdc_peer_copy(wdc_context* dst_ctx, void* dst, wdc_context* src_ctx, const void* src,
                             int64_t bytes) {
  if (!dst_ctx || !src_ctx || bytes < 0 || (bytes > 0 && (!dst || !src)))
    return wdc_fail(dst_ctx, WDC_ERR_INVALID, "wdc_peer_copy: bad argument");
  wdc_note_write(dst_ctx, dst, bytes);
  if (bytes == 0) return WDC_OK;
  // Order the copy after everything already enqueued on the source stream, run it on the
  // destination stream.
  cudaEvent_t ev;
  {
    DeviceGuard g(src_ctx->device);
    WDC_CUDA(src_ctx, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    WDC_CUDA(src_ctx, cudaEventRecord(ev, src_ctx->stream));
  }
  DeviceGuard g(dst_ctx->device);
  WDC_CUDA(dst_ctx, cudaStreamWaitEvent(dst_ctx->stream, ev, 0));
  WDC_CUDA(dst_ctx, cudaMemcpyPeerAsync(dst, dst_ctx->device, src, src_ctx->device, (size_t)bytes,
                                        dst_ctx->stream));
  // the source must not reuse the buffer before the copy has read it
  cudaEvent_t done;
  WDC_CUDA(dst_ctx, cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
  WDC_CUDA(dst_ctx, cudaEventRecord(done, dst_ctx->stream));
  {
    DeviceGuard g2(src_ctx->device);
    WDC_CUDA(src_ctx, cudaStreamWaitEvent(src_ctx->stream, done, 0));
  }
  cudaEventDestroy(ev);
  cudaEventDestroy(done);
  return WDC_OK;
}
