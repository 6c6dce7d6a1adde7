// Host side of libbikv.so: argument checking, plan building/validation,
// launch configuration and the peer / IPC plumbing.  See include/bikv.h for the
// contract of every entry point.
#include "bikv_kernels.cuh"

#include <algorithm>
#include <atomic>
#include <cstring>
#include <mutex>
#include <vector>

namespace {

using namespace bikv;

thread_local int tl_cuda_error = 0;
std::atomic<long long> g_launches{0};

// Tuning knobs (plain atomics: readers take a snapshot per call).
// ld/st kernels: enough CTAs that every warp takes ONE chunk (the cap is far above what a launch
// asks for) and small chunks -- the hardware's block scheduler then balances the work, where a
// grid-stride loop over 16 CTAs per SM left a tail: 1.036 of the measured HBM copy peak against
// 1.000 at config 1 (4 KiB chunks, uncapped grid, 32-byte accesses), 0.866 with 2 KiB chunks.
std::atomic<long long> g_ldst_ctas_per_sm{4096};
std::atomic<long long> g_ldst_seg_bytes{4096};
std::atomic<long long> g_bulk_ctas_per_sm{3};
std::atomic<long long> g_bulk_stages{4};
std::atomic<long long> g_seg_bytes{16384};
std::atomic<long long> g_ldst_wide{1};     // 1: 32-byte ld/st in k_paged_ldst and k_flat where alignment allows
std::atomic<long long> g_bulk_span{1};     // adjacent planes of a page per stage of the bulk ring
std::atomic<long long> g_auto_variant{0};  // 0 = choose by shard count
std::atomic<long long> g_tm_threads{0};        // CTA size of k_token_major16v; 0 = by tile size (see launcher)
std::atomic<long long> g_ldst_threads{256};    // CTA size of k_paged_ldst (k_paged_nhd and k_flat use 256)
std::atomic<long long> g_tm16_threads{256};    // CTA size of k_token_major16
std::atomic<long long> g_tm_max_groups{16};    // cap on d-groups per slab (k_token_major16v)
std::atomic<long long> g_tm_tile_kib{48};      // cap on one slab tile of k_token_major16v holding all heads, KiB
std::atomic<long long> g_tm_split_tile_kib{96};  // the same for a slab that splits the heads
std::atomic<long long> g_tm_scatter_staged{1};  // k_token_major16v scatter: 1 = through staged worker rows, 0 = through the transposed tile
std::atomic<long long> g_tm_gather_stages{0};   // buffers in the gather's cp.async ring of k_token_major16v: 2, 3, 0 = by tile size
std::atomic<long long> g_tm_scatter_stages{2};  // the same for the staged scatter
std::atomic<long long> g_tm_max_heads{64};
std::atomic<long long> g_tm_single{1};         // k_token_major16v: 1 = one item per CTA, no ring (0 = persistent CTAs with a cp.async ring)     // cap on heads per slab when the slab splits the heads

int cuda_fail(cudaError_t e) {
  tl_cuda_error = (int)e;
  return BIKV_ERR_CUDA;
}
#define BIKV_CUDA(expr)                                \
  do {                                                 \
    cudaError_t e__ = (expr);                          \
    if (e__ != cudaSuccess) return cuda_fail(e__);     \
  } while (0)

struct DeviceInfo {
  int sm_count = 0;
  int max_optin_smem = 0;
};
std::mutex g_dev_mu;
DeviceInfo g_dev[64];
bool g_dev_known[64] = {false};

int device_info(DeviceInfo* out) {
  int dev = 0;
  BIKV_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return BIKV_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lk(g_dev_mu);
  if (!g_dev_known[dev]) {
    BIKV_CUDA(cudaDeviceGetAttribute(&g_dev[dev].sm_count, cudaDevAttrMultiProcessorCount, dev));
    BIKV_CUDA(cudaDeviceGetAttribute(&g_dev[dev].max_optin_smem,
                                     cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    g_dev_known[dev] = true;
  }
  *out = g_dev[dev];
  return BIKV_OK;
}

int check_geometry(const bikv_geometry* g) {
  if (!g) return BIKV_ERR_BAD_ARG;
  if (g->n_layers <= 0 || g->n_kv_heads <= 0 || g->head_dim <= 0 || g->page_tokens <= 0)
    return BIKV_ERR_BAD_ARG;
  if (g->elt_bytes != 1 && g->elt_bytes != 2 && g->elt_bytes != 4) return BIKV_ERR_BAD_ARG;
  if (g->pool_layout != BIKV_POOL_PAGED && g->pool_layout != BIKV_POOL_TOKEN_MAJOR)
    return BIKV_ERR_BAD_ARG;
  const long long row = (long long)g->n_kv_heads * g->head_dim * g->elt_bytes;
  if (g->pool_layout == BIKV_POOL_PAGED) {
    if (row % 16 != 0) return BIKV_ERR_ALIGNMENT;
  } else {
    // 16-byte worker vectors run along dim.
    if (((long long)g->head_dim * g->elt_bytes) % 16 != 0) return BIKV_ERR_ALIGNMENT;
  }
  if (row * g->page_tokens > (1ll << 30)) return BIKV_ERR_TOO_LARGE;
  return BIKV_OK;
}

int check_pool(const bikv_pool_desc* p) {
  if (!p) return BIKV_ERR_BAD_ARG;
  if (p->n_shards <= 0 || p->n_shards > BIKV_MAX_SHARDS) return BIKV_ERR_BAD_ARG;
  if (p->pages_per_shard <= 0) return BIKV_ERR_BAD_ARG;
  if (p->shard_rule != BIKV_SHARD_MOD && p->shard_rule != BIKV_SHARD_BLOCK) return BIKV_ERR_BAD_ARG;
  if (p->pages_per_shard * p->n_shards > 0x7fffffffll) return BIKV_ERR_TOO_LARGE;
  for (int s = 0; s < p->n_shards; ++s) {
    if (!p->shard_base[s]) return BIKV_ERR_BAD_ARG;
    if (((uintptr_t)p->shard_base[s]) & 15) return BIKV_ERR_ALIGNMENT;
  }
  return BIKV_OK;
}

PoolDev to_dev(const bikv_pool_desc* p) {
  PoolDev d;
  memset(&d, 0, sizeof(d));
  for (int s = 0; s < p->n_shards; ++s) d.base[s] = (char*)p->shard_base[s];
  d.n_shards = p->n_shards;
  d.rule = p->shard_rule;
  d.pages_per_shard = p->pages_per_shard;
  return d;
}

int after_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return BIKV_OK;
}

FastDiv fast_div(unsigned d) {
  FastDiv f;
  f.d = d;
  f.m = d == 1 ? 0u : (unsigned)((1ull << 32) / d + 1);
  return f;
}

// Token-major pool with 2-byte elements and head_dim a multiple of 8.
int launch_token_major16(const bikv_pool_desc* pool, const bikv_geometry* g, const bikv_page_rec* recs,
                         long long n_pages, const bikv_request_desc* reqs, int to_pool, cudaStream_t st,
                         const DeviceInfo& di, int32_t* status, int32_t n_requests) {
  const unsigned H = g->n_kv_heads, D = g->head_dim, L = g->n_layers;
  const unsigned G = D / 8;
  const unsigned Lp = L | 1u;
  // Largest slab (Gs groups of 8 d) that divides G and keeps the tile within the
  // budget below, so that a few CTAs share an SM and cover each other's phases.
  const long long per_group = 8ll * H * Lp * 4;
  const long long budget = std::min<long long>(di.max_optin_smem, 100 * 1024);
  unsigned Gs = 0;
  for (unsigned cand = G; cand >= 1; --cand) {
    if (G % cand) continue;
    if (per_group * cand <= budget) {
      Gs = cand;
      break;
    }
  }
  if (Gs == 0) {
    Gs = 1;
    if (per_group > di.max_optin_smem) return BIKV_ERR_TOO_LARGE;
  }
  const long long smem = per_group * Gs;
  const long long items = n_pages * g->page_tokens * (long long)(G / Gs);
  if (items > 0x7fffffffll) return BIKV_ERR_TOO_LARGE;
  TokenMajor16Args a;
  memset(&a, 0, sizeof(a));
  a.recs = reinterpret_cast<const uint4*>(recs);
  a.reqs = reqs;
  a.pool = to_dev(pool);
  a.n_items = (unsigned)items;
  a.page_tokens = g->page_tokens;
  a.slabs = G / Gs;
  a.Gs = Gs;
  a.H = H;
  a.D = D;
  a.L = L;
  a.Lp = Lp;
  a.token_bytes = (unsigned long long)D * H * L * 4ull;
  a.to_pool = to_pool;
  a.status = status;
  a.n_requests = (unsigned)n_requests;
  a.total_pages = (unsigned long long)pool->pages_per_shard * pool->n_shards;
  a.div_L = fast_div(L);
  a.div_H = fast_div(H);
  a.div_HG = fast_div(H * Gs);
  a.div_Gs = fast_div(Gs);
  a.div_slabs = fast_div(a.slabs);
  a.div_ptok = fast_div((unsigned)g->page_tokens);
  // FastDiv is exact while dividend * divisor < 2^32.
  if ((unsigned long long)items * std::max<unsigned>(a.slabs, (unsigned)g->page_tokens) >= (1ull << 32) ||
      (unsigned long long)(Gs * 8ull * H * L) * std::max(L, H * Gs) >= (1ull << 32))
    return BIKV_ERR_TOO_LARGE;
  const unsigned grid = (unsigned)items;      // one item per CTA: the block scheduler balances the launch
  if (grid == 0) return BIKV_OK;
  if (smem > 40 * 1024)
    BIKV_CUDA(cudaFuncSetAttribute(k_token_major16, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  BIKV_CUDA(cudaFuncSetAttribute(k_token_major16, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared));
  k_token_major16<<<grid, (unsigned)g_tm16_threads.load() / 32 * 32, (size_t)smem, st>>>(a);
  return after_launch();
}


// Token-major pool, 2-byte elements, head_dim % 8 == 0 and n_layers % 4 == 0.
// Returns 1 if the geometry does not fit this kernel (caller falls back).
int launch_token_major16v(const bikv_pool_desc* pool, const bikv_geometry* g, const bikv_page_rec* recs,
                          long long n_pages, const bikv_request_desc* reqs, int to_pool, cudaStream_t st,
                          const DeviceInfo& di, int32_t* status, int32_t n_requests) {
  const unsigned H = g->n_kv_heads, D = g->head_dim, L = g->n_layers;
  const unsigned G = D / 8, LU = L / 4;
  const unsigned RU = std::max(8u, (LU + 7u) & ~7u);   // row pitch in 16-byte units
  const long long per_gh = 8ll * 16ll * RU;            // tile bytes per (d-group, head)
  const unsigned max_groups = (unsigned)std::max<long long>(1, g_tm_max_groups.load());
  // Slab = Gs d-groups x Hs heads.  All heads within 48 KiB when that leaves worker-side runs
  // (Gs*16 bytes per head) of 128 bytes or more; otherwise the most heads that do within
  // 96 KiB.  Measured at 80 layers x 8 heads, fractions of the HBM copy peak: 4 heads x 64 d
  // (96 KiB) 0.83-0.85, 1 head x 128 d (48 KiB) 0.77, 2 heads x 64 d (48 KiB) 0.73,
  // 1 head x 64 d (24 KiB) 0.62; the older kernel 0.61.
  const long long cap_all = g_tm_tile_kib.load() * 1024, cap_split = g_tm_split_tile_kib.load() * 1024;
  unsigned Gs = 0, Hs = 0;
  const unsigned max_split_heads = (unsigned)std::max<long long>(1, g_tm_max_heads.load());
  for (unsigned hs = H; hs >= 1 && Gs == 0; --hs) {
    if (H % hs || (hs < H && hs > max_split_heads)) continue;
    for (unsigned cand = std::min(G, max_groups); cand >= 1; --cand) {
      if (G % cand) continue;
      if (per_gh * hs * cand <= (hs == H ? cap_all : cap_split)) {
        if (cand >= 8) { Gs = cand; Hs = hs; }
        break;
      }
    }
  }
  // No slab with 128-byte runs (head_dim below 64, or rows too long): the older kernel,
  // whose slab may hold more d-groups, does better there.
  if (Gs == 0) return 1;
  const long long tile = per_gh * Hs * Gs;
  const bool staged = to_pool && g_tm_scatter_staged.load() != 0;
  const long long stage = 8ll * LU * ((Hs * Gs + 7u) & ~7u) * 16;   // the slab's worker vectors, unpadded
  // Ring depth: three buffers for tiles up to 48 KiB (gather at 28 layers: 0.92-0.93 of the HBM
  // copy peak with 3 x 256 threads against 0.87-0.88 with 2 x 64); larger tiles keep two (three
  // smaller ones measured 0.73-0.76 against 0.92 at 80 layers x 8 heads).
  const long long unit = staged ? stage : tile;
  long long stages = (to_pool ? g_tm_scatter_stages : g_tm_gather_stages).load();
  if (stages == 0) stages = tile <= 48 * 1024 ? 3 : 2;
  if (stages < 2) stages = 2;
  if (stages * unit > di.max_optin_smem) stages = 2;
  const bool single = g_tm_single.load() != 0 && !(to_pool && !staged);
  const long long smem = (to_pool && !staged) ? tile : (single ? unit : stages * unit);
  if (smem > di.max_optin_smem) return 1;
  const unsigned slabs = (G / Gs) * (H / Hs);
  const long long items = n_pages * g->page_tokens * (long long)slabs;
  if (items > 0x7fffffffll) return BIKV_ERR_TOO_LARGE;
  const unsigned long long rows = 8ull * Gs * Hs;
  // FastDiv is exact while dividend * divisor < 2^32.
  if ((unsigned long long)items * std::max<unsigned>(slabs, (unsigned)g->page_tokens) >= (1ull << 32) ||
      rows * LU * std::max(std::max(LU, Hs), Hs * Gs) >= (1ull << 32))
    return BIKV_ERR_TOO_LARGE;
  TokenMajor16vArgs a;
  memset(&a, 0, sizeof(a));
  a.recs = reinterpret_cast<const uint4*>(recs);
  a.reqs = reqs;
  a.pool = to_dev(pool);
  a.n_items = (unsigned)items;
  a.page_tokens = g->page_tokens;
  a.slabs = slabs;
  a.hslabs = H / Hs;
  a.Gs = Gs;
  a.Hs = Hs;
  a.H = H;
  a.D = D;
  a.L = L;
  a.LU = LU;
  a.RU = RU;
  a.d_skip = (H - Hs) * LU;
  a.div_LU = fast_div(LU);
  a.div_Hs = fast_div(Hs);
  a.div_HG = fast_div(Hs * Gs);
  a.div_Gs = fast_div(Gs);
  a.div_slabs = fast_div(a.slabs);
  a.div_hslabs = fast_div(a.hslabs);
  a.div_ptok = fast_div((unsigned)g->page_tokens);
  a.token_bytes = (unsigned long long)D * H * L * 4ull;
  a.to_pool = to_pool;
  a.status = status;
  a.n_requests = (unsigned)n_requests;
  a.total_pages = (unsigned long long)pool->pages_per_shard * pool->n_shards;
  const long long per_sm = std::max<long long>(1, std::min<long long>(12, (220 * 1024) / (smem + 1024)));
  a.single = single ? 1 : 0;
  const unsigned grid = single ? (unsigned)items : (unsigned)std::min<long long>(items, (long long)di.sm_count * per_sm);
  if (grid == 0) return BIKV_OK;
  const int mode = staged ? 2 : (to_pool ? 1 : 0);
  const bool ring3 = mode != 1 && stages == 3;
  void (*kern)(TokenMajor16vArgs) = nullptr;
  if (Hs < H) {
    kern = mode == 1 ? k_token_major16v<true, 1, false>
           : mode == 2 ? (ring3 ? k_token_major16v<true, 2, true> : k_token_major16v<true, 2, false>)
                       : (ring3 ? k_token_major16v<true, 0, true> : k_token_major16v<true, 0, false>);
  } else {
    kern = mode == 1 ? k_token_major16v<false, 1, false>
           : mode == 2 ? (ring3 ? k_token_major16v<false, 2, true> : k_token_major16v<false, 2, false>)
                       : (ring3 ? k_token_major16v<false, 0, true> : k_token_major16v<false, 0, false>);
  }
  BIKV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)std::max<long long>(smem, 48 * 1024)));
  BIKV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared));
  // CTA size, by measurement (fractions of the HBM copy peak).  Tiles up to 48 KiB (28 layers,
  // 2 or 4 heads): gather with three tiles 0.92-0.93 with 256 threads, 0.90 with 128, 0.82-0.83
  // with 64; with two tiles 0.87-0.88 with 64, 0.85 with 96-128, 0.81 with 224-256; staged scatter 0.92-0.94 with 64, 0.90-0.91 with 96, 0.88-0.91 with 128, 0.77-0.80 with 32.
  // 96 KiB tiles (80 layers x 8 heads): gather 0.912 / 0.923 / 0.916 with 128 / 192 / 256;
  // staged scatter 0.916 / 0.963 / 0.970 / 0.957 with 128 / 192 / 224 / 256; the scatter
  // through the transposed tile 0.753 / 0.766 / 0.786 with 128 / 192 / 256.
  // One item per CTA (the default): 0.98-0.99 / 1.01 gather / scatter for 28 layers x 2 or 4 heads and 1.00 / 1.00
  // for 80 layers x 8 heads, against 0.92-0.94 / 0.93-0.98 for the persistent ring -- the CTAs that share an
  // SM cover each other's latencies and the block scheduler balances the launch.  Gather with 128 or 64 threads
  // 0.984-0.990, with 256 0.78; scatter with 64 threads 1.007, with 256 0.87.
  unsigned threads = (unsigned)g_tm_threads.load();
  if (threads == 0 && single)
    threads = to_pool ? (tile <= 48 * 1024 ? 64 : 224) : (tile <= 48 * 1024 ? 128 : 192);
  if (threads == 0) {
    if (to_pool)
      threads = staged ? (tile <= 48 * 1024 ? 64 : 224) : (tile <= 48 * 1024 ? 128 : 256);
    else
      threads = stages == 3 ? 256 : (tile <= 48 * 1024 ? 64 : 192);
  }
  threads = std::min(256u, std::max(32u, threads & ~31u));
  kern<<<grid, threads, (size_t)smem, st>>>(a);
  return after_launch();
}

int launch_token_major(const bikv_pool_desc* pool, const bikv_geometry* g, const bikv_page_rec* recs,
                       long long n_pages, const bikv_request_desc* reqs, int to_pool,
                       cudaStream_t st, int32_t* status, int32_t n_requests) {
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc) return rc;
  if (g->elt_bytes == 2 && g->head_dim % 8 == 0 && g->n_layers % 4 == 0) {
    rc = launch_token_major16v(pool, g, recs, n_pages, reqs, to_pool, st, di, status, n_requests);
    if (rc != 1) return rc;
  }
  if (g->elt_bytes == 2 && g->head_dim % 8 == 0)
    return launch_token_major16(pool, g, recs, n_pages, reqs, to_pool, st, di, status, n_requests);
  const unsigned V = 16 / g->elt_bytes;
  const unsigned C = 2u * g->n_layers;
  const unsigned H = g->n_kv_heads, D = g->head_dim;
  // Largest slab (DT d-values) that divides D, is a multiple of V and stays
  // within 48 KiB of shared memory so several CTAs share an SM.
  const long long per_d = (long long)H * C * g->elt_bytes;
  unsigned DT = 0;
  for (unsigned cand = D; cand >= V; --cand) {
    if (D % cand || cand % V) continue;
    if (per_d * cand <= 48 * 1024) {
      DT = cand;
      break;
    }
  }
  if (DT == 0) {
    // Even one vector of d exceeds 48 KiB: take the opt-in limit.
    DT = V;
    if (per_d * DT > di.max_optin_smem) return BIKV_ERR_TOO_LARGE;
  }
  const long long smem = per_d * DT;
  const long long items = n_pages * g->page_tokens * (long long)(D / DT);
  if (items > 0x7fffffffll) return BIKV_ERR_TOO_LARGE;
  TokenMajorArgs a;
  memset(&a, 0, sizeof(a));
  a.recs = reinterpret_cast<const uint4*>(recs);
  a.reqs = reqs;
  a.pool = to_dev(pool);
  a.n_items = (unsigned)items;
  a.page_tokens = g->page_tokens;
  a.slabs = D / DT;
  a.DT = DT;
  a.H = H;
  a.D = D;
  a.C = C;
  a.token_bytes = (unsigned long long)per_d * D;
  a.to_pool = to_pool;
  a.status = status;
  a.n_requests = (unsigned)n_requests;
  a.total_pages = (unsigned long long)pool->pages_per_shard * pool->n_shards;
  const int threads = 256;
  unsigned grid = (unsigned)items;            // one item per CTA
  if (grid == 0) return BIKV_OK;
  auto launch = [&](auto kern) -> int {
    if (smem > 48 * 1024)
      BIKV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, threads, (size_t)smem, st>>>(a);
    return after_launch();
  };
  switch (g->elt_bytes) {
    case 1: return launch(k_token_major<uint8_t>);
    case 2: return launch(k_token_major<uint16_t>);
    default: return launch(k_token_major<uint32_t>);
  }
}

int launch_paged(const bikv_pool_desc* pool, const bikv_geometry* g, const bikv_page_rec* recs,
                 long long n_pages, const bikv_request_desc* reqs, int to_pool, int variant,
                 int32_t* status, cudaStream_t st, int32_t n_requests) {
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc) return rc;
  // AUTO: ld/st when every page is local (0.97-0.99 of HBM copy bandwidth there, the
  // bulk ring 0.93); the bulk ring when shards are peer mappings (its larger requests
  // load NVLink better: 652 vs 626 GB/s per GPU measured on 8 GPUs).
  if (variant == BIKV_VARIANT_AUTO)
    variant = g_auto_variant.load() ? (int)g_auto_variant.load()
                                    : (pool->n_shards > 1 ? BIKV_VARIANT_BULK : BIKV_VARIANT_LDST);
  if (variant != BIKV_VARIANT_LDST && variant != BIKV_VARIANT_BULK) return BIKV_ERR_BAD_ARG;
  if (variant == BIKV_VARIANT_BULK && !status) return BIKV_ERR_BAD_ARG;

  PagedArgs a;
  memset(&a, 0, sizeof(a));
  a.recs = reinterpret_cast<const uint4*>(recs);
  a.reqs = reqs;
  a.pool = to_dev(pool);
  a.planes = 2u * g->n_layers;
  a.row_bytes = (unsigned)(g->n_kv_heads * g->head_dim * g->elt_bytes);
  a.plane_bytes = a.row_bytes * g->page_tokens;
  a.page_bytes = (unsigned long long)a.plane_bytes * a.planes;
  // Chunk size: small for the ld/st kernel (one chunk per warp), a plane for the bulk ring.
  unsigned seg = (unsigned)(variant == BIKV_VARIANT_LDST ? g_ldst_seg_bytes : g_seg_bytes).load();
  if (seg > a.plane_bytes) seg = a.plane_bytes;  // plane_bytes is a multiple of 16
  a.seg_bytes = seg;
  a.parts = (a.plane_bytes + seg - 1) / seg;
  const long long items = n_pages * (long long)a.planes * a.parts;
  if (items > 0x7fffffffll) return BIKV_ERR_TOO_LARGE;
  a.n_items = (unsigned)items;
  a.to_pool = to_pool;
  a.status = status;
  a.n_requests = (unsigned)n_requests;
  a.page_tokens = (unsigned)g->page_tokens;
  a.total_pages = (unsigned long long)pool->pages_per_shard * pool->n_shards;
  a.wide = (int)g_ldst_wide.load();
  if (items == 0) return BIKV_OK;

  if (variant == BIKV_VARIANT_LDST) {
    const int threads = (int)g_ldst_threads.load() / 32 * 32, warps = threads / 32;
    const long long want = (items + warps - 1) / warps;
    unsigned grid = (unsigned)std::min<long long>(want, (long long)di.sm_count * g_ldst_ctas_per_sm.load());
    k_paged_ldst<8><<<grid, threads, 0, st>>>(a);
    return after_launch();
  }
  int stages = (int)g_bulk_stages.load();
  long long per_sm = g_bulk_ctas_per_sm.load();
  // Adjacent planes per ring stage ("bulk_span").  Only when a stage holds whole planes.
  unsigned span = (unsigned)g_bulk_span.load();
  if (a.parts != 1 || span > a.planes) span = a.parts != 1 ? 1u : a.planes;
  const long long budget = std::min<long long>(di.max_optin_smem, 227 * 1024) - 1024;
  while (span > 1 && 2ll * seg * span > budget) --span;   // at least two stages must fit
  a.span = span;
  a.groups = (a.planes + span - 1) / span;
  if (span > 1) a.n_items = (unsigned)(n_pages * (long long)a.groups);   // fewer than `items`, which fitted
  const long long stage_bytes = (long long)seg * span;
  while (stages > 2 && (long long)stages * stage_bytes > budget) --stages;
  if ((long long)stages * stage_bytes > budget) return BIKV_ERR_TOO_LARGE;
  const long long smem = (long long)stages * stage_bytes;
  while (per_sm > 1 && per_sm * (smem + 1024) > 227 * 1024) --per_sm;
  unsigned grid = (unsigned)std::min<long long>(a.n_items, (long long)di.sm_count * per_sm);
  // The kernel also holds a few static bytes (its mbarriers), so opt in well
  // before the 48 KiB default limit.
  if (smem > 40 * 1024)
    BIKV_CUDA(cudaFuncSetAttribute(k_paged_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  k_paged_bulk<<<grid, 32, (size_t)smem, st>>>(a, stages);
  return after_launch();
}

int run(const bikv_pool_desc* pool, const bikv_geometry* geom, const bikv_page_rec* recs_dev,
        int64_t n_pages, const bikv_request_desc* reqs_dev, int32_t n_requests, int to_pool,
        int variant, int32_t* status_dev, void* stream) {
  int rc = check_geometry(geom);
  if (rc) return rc;
  rc = check_pool(pool);
  if (rc) return rc;
  if (n_pages < 0 || n_requests < 0) return BIKV_ERR_BAD_ARG;
  if (n_pages == 0) return BIKV_OK;
  if (!recs_dev || !reqs_dev || n_requests == 0) return BIKV_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (geom->pool_layout == BIKV_POOL_TOKEN_MAJOR)
    return launch_token_major(pool, geom, recs_dev, n_pages, reqs_dev, to_pool, st, status_dev, n_requests);
  return launch_paged(pool, geom, recs_dev, n_pages, reqs_dev, to_pool, variant, status_dev, st, n_requests);
}

int run_h(const bikv_pool_desc* pool, const bikv_geometry* geom, const bikv_page_rec* recs_host,
          int64_t n_pages, const bikv_request_desc* reqs_host, int32_t n_requests, void* scratch,
          int64_t scratch_bytes, int validate, int to_pool, int variant, int32_t* status_dev,
          void* stream) {
  if (n_pages < 0 || n_requests < 0) return BIKV_ERR_BAD_ARG;
  if (n_pages == 0) return BIKV_OK;
  if (!recs_host || !reqs_host || !scratch) return BIKV_ERR_BAD_ARG;
  for (int32_t r = 0; r < n_requests; ++r)
    if (!reqs_host[r].base) return BIKV_ERR_BAD_ARG;
  if (validate) {
    int rc = bikv_plan_validate(recs_host, n_pages, reqs_host, n_requests, pool, geom, to_pool);
    if (rc) return rc;
  }
  const int64_t need = bikv_plan_scratch_bytes(n_pages, n_requests);
  if (scratch_bytes < need) return BIKV_ERR_TOO_LARGE;
  if (((uintptr_t)scratch) & 15) return BIKV_ERR_ALIGNMENT;
  cudaStream_t st = (cudaStream_t)stream;
  char* d_recs = (char*)scratch;
  const size_t rec_bytes = (size_t)n_pages * sizeof(bikv_page_rec);
  char* d_reqs = d_recs + ((rec_bytes + 255) & ~(size_t)255);
  BIKV_CUDA(cudaMemcpyAsync(d_recs, recs_host, rec_bytes, cudaMemcpyHostToDevice, st));
  BIKV_CUDA(cudaMemcpyAsync(d_reqs, reqs_host, (size_t)n_requests * sizeof(bikv_request_desc),
                            cudaMemcpyHostToDevice, st));
  return run(pool, geom, (const bikv_page_rec*)d_recs, n_pages, (const bikv_request_desc*)d_reqs,
             n_requests, to_pool, variant, status_dev, stream);
}

struct Knob {
  const char* name;
  std::atomic<long long>* v;
  long long lo, hi;
};
Knob* find_knob(const char* name) {
  static Knob knobs[] = {
      {"ldst_ctas_per_sm", &g_ldst_ctas_per_sm, 1, 4096},
      {"bulk_ctas_per_sm", &g_bulk_ctas_per_sm, 1, 16},
      {"bulk_stages", &g_bulk_stages, 2, kMaxStages},
      {"seg_bytes", &g_seg_bytes, 1024, 64 * 1024},
      {"ldst_seg_bytes", &g_ldst_seg_bytes, 1024, 64 * 1024},
      {"bulk_span", &g_bulk_span, 1, 8},
      {"ldst_wide", &g_ldst_wide, 0, 1},
      {"auto_variant", &g_auto_variant, 0, BIKV_VARIANT_BULK},
      {"ldst_threads", &g_ldst_threads, 64, 256},
      {"tm_threads", &g_tm_threads, 0, 256},
      {"tm16_threads", &g_tm16_threads, 64, 256},
      {"tm_max_groups", &g_tm_max_groups, 1, 64},
      {"tm_tile_kib", &g_tm_tile_kib, 8, 100},
      {"tm_split_tile_kib", &g_tm_split_tile_kib, 8, 100},
      {"tm_max_heads", &g_tm_max_heads, 1, 64},
      {"tm_single", &g_tm_single, 0, 1},
      {"tm_scatter_staged", &g_tm_scatter_staged, 0, 1},
      {"tm_gather_stages", &g_tm_gather_stages, 0, 3},
      {"tm_scatter_stages", &g_tm_scatter_stages, 0, 3},
  };
  if (!name) return nullptr;
  for (auto& k : knobs)
    if (!strcmp(k.name, name)) return &k;
  return nullptr;
}

}  // namespace

extern "C" {

int bikv_version(void) { return BIKV_ABI_VERSION; }

const char* bikv_strerror(int status) {
  switch (status) {
    case BIKV_OK: return "ok";
    case BIKV_ERR_BAD_ARG: return "bad argument";
    case BIKV_ERR_PAGE_RANGE: return "page id outside the pool";
    case BIKV_ERR_DST_RANGE: return "token window outside the request tensor";
    case BIKV_ERR_ALIGNMENT: return "address or row not 16-byte aligned";
    case BIKV_ERR_PEER: return "peer access or IPC mapping unavailable";
    case BIKV_ERR_CUDA: return "CUDA call failed (see bikv_last_cuda_error)";
    case BIKV_ERR_OVERLAP: return "scatter plan names a pool page twice";
    case BIKV_ERR_DEVICE_TIMEOUT: return "bounded device wait ran out";
    case BIKV_ERR_TOO_LARGE: return "size beyond a documented maximum";
    case BIKV_ERR_PLAN: return "inconsistent plan";
    default: return "unknown status";
  }
}

int bikv_last_cuda_error(void) { return tl_cuda_error; }
int64_t bikv_launch_count(void) { return g_launches.load(); }

int bikv_set_tuning(const char* name, int64_t value) {
  Knob* k = find_knob(name);
  if (!k || value < k->lo || value > k->hi) return BIKV_ERR_BAD_ARG;
  if ((!strcmp(name, "seg_bytes") || !strcmp(name, "ldst_seg_bytes")) && (value % 1024) != 0) return BIKV_ERR_BAD_ARG;
  k->v->store(value);
  return BIKV_OK;
}
int64_t bikv_get_tuning(const char* name) {
  Knob* k = find_knob(name);
  return k ? k->v->load() : (int64_t)BIKV_ERR_BAD_ARG;
}

int64_t bikv_plan_build(const int32_t* pages_flat, const int64_t* item_page_begin,
                        const int32_t* item_tokens, const int32_t* item_request,
                        const int32_t* item_shard, int64_t pages_per_shard, int32_t n_items,
                        int32_t page_tokens, int64_t* request_tokens, int32_t n_requests,
                        bikv_page_rec* out, int64_t out_capacity) {
  if (n_items < 0 || page_tokens <= 0 || n_requests <= 0) return BIKV_ERR_BAD_ARG;
  if (n_items == 0) return 0;
  if (!item_page_begin || !item_tokens || !request_tokens || !out) return BIKV_ERR_BAD_ARG;
  if (item_shard && pages_per_shard <= 0) return BIKV_ERR_BAD_ARG;
  int64_t n = 0;
  for (int32_t it = 0; it < n_items; ++it) {
    const int64_t b = item_page_begin[it], e = item_page_begin[it + 1];
    if (b < 0 || e < b) return BIKV_ERR_PLAN;
    const int32_t req = item_request ? item_request[it] : 0;
    if (req < 0 || req >= n_requests) return BIKV_ERR_BAD_ARG;
    const int32_t tokens = item_tokens[it];
    if (tokens < 0) return BIKV_ERR_PLAN;
    if (e > b && !pages_flat) return BIKV_ERR_BAD_ARG;
    const int32_t rem = tokens % page_tokens;
    for (int64_t p = b; p < e; ++p) {
      // Tail rule of the reference: only the LAST page of an item is short,
      // and only when the token count is not a multiple of the page size.
      const int32_t size = (p == e - 1 && rem != 0) ? rem : page_tokens;
      if (n >= out_capacity) return BIKV_ERR_TOO_LARGE;
      const int64_t off = request_tokens[req];
      if (off > 0x7fffffffll - size) return BIKV_ERR_TOO_LARGE;
      int64_t id = pages_flat[p];
      if (item_shard) {
        if (id < 0 || id >= pages_per_shard) return BIKV_ERR_PAGE_RANGE;
        id += (int64_t)item_shard[it] * pages_per_shard;
        if (id > 0x7fffffffll) return BIKV_ERR_TOO_LARGE;
      }
      out[n].page_id = (int32_t)id;
      out[n].valid_tokens = size;
      out[n].request = req;
      out[n].token_offset = (int32_t)off;
      request_tokens[req] = off + size;
      ++n;
    }
  }
  return n;
}

int64_t bikv_plan_split_by_owner(const bikv_page_rec* const* tables, const int64_t* n_rows,
                                 const int32_t* requests_per_worker, int32_t n_workers, int32_t owner,
                                 int32_t n_shards, int64_t pages_per_shard, int32_t shard_rule,
                                 bikv_page_rec* out, int64_t out_capacity) {
  if (n_workers < 0 || n_shards <= 0 || owner < 0 || owner >= n_shards || pages_per_shard <= 0 || out_capacity < 0)
    return BIKV_ERR_BAD_ARG;
  if (shard_rule != BIKV_SHARD_MOD && shard_rule != BIKV_SHARD_BLOCK) return BIKV_ERR_BAD_ARG;
  if (n_workers == 0) return 0;
  if (!tables || !n_rows || !requests_per_worker || (!out && out_capacity > 0)) return BIKV_ERR_BAD_ARG;
  // Pass 1: this owner's rows per worker.  Pass 2: merge the workers' sequences by the
  // position (i + 1/2) / n of a row within its worker's n rows, ties to the lower worker, so
  // that the destinations interleave in proportion and a worker's rows keep their order.
  std::vector<std::vector<int64_t>> mine((size_t)n_workers);
  int64_t total = 0;
  for (int32_t w = 0; w < n_workers; ++w) {
    if (n_rows[w] < 0 || (n_rows[w] > 0 && !tables[w])) return BIKV_ERR_BAD_ARG;
    for (int64_t i = 0; i < n_rows[w]; ++i) {
      const int64_t id = tables[w][i].page_id;
      if (id < 0) return BIKV_ERR_PAGE_RANGE;
      const int64_t shard = shard_rule == BIKV_SHARD_MOD ? id % n_shards : id / pages_per_shard;
      if (shard >= n_shards) return BIKV_ERR_PAGE_RANGE;
      if (shard == owner) mine[(size_t)w].push_back(i);
    }
    total += (int64_t)mine[(size_t)w].size();
  }
  if (total > out_capacity) return BIKV_ERR_TOO_LARGE;
  std::vector<int64_t> base((size_t)n_workers, 0), at((size_t)n_workers, 0);
  for (int32_t w = 1; w < n_workers; ++w) {
    if (requests_per_worker[w - 1] < 0) return BIKV_ERR_BAD_ARG;
    base[(size_t)w] = base[(size_t)w - 1] + requests_per_worker[w - 1];
  }
  for (int64_t k = 0; k < total; ++k) {
    int32_t best = -1;
    for (int32_t w = 0; w < n_workers; ++w) {
      const int64_t n = (int64_t)mine[(size_t)w].size();
      if (at[(size_t)w] >= n) continue;
      if (best < 0) {
        best = w;
        continue;
      }
      // (2*at_w + 1) / n_w  <  (2*at_b + 1) / n_b   compared without division
      const int64_t nb = (int64_t)mine[(size_t)best].size();
      if ((__int128)(2 * at[(size_t)w] + 1) * nb < (__int128)(2 * at[(size_t)best] + 1) * n) best = w;
    }
    bikv_page_rec r = tables[best][mine[(size_t)best][(size_t)at[(size_t)best]++]];
    const int64_t req = (int64_t)r.request + base[(size_t)best];
    if (r.request < 0 || r.request >= requests_per_worker[best] || req > 0x7fffffffll) return BIKV_ERR_BAD_ARG;
    r.request = (int32_t)req;
    out[k] = r;
  }
  return total;
}

int bikv_check_worker_base(const void* base) {
  return worker_base_status((unsigned long long)(uintptr_t)base);
}

int bikv_plan_validate(const bikv_page_rec* recs, int64_t n_pages, const bikv_request_desc* requests,
                       int32_t n_requests, const bikv_pool_desc* pool, const bikv_geometry* geom,
                       int check_overlap) {
  int rc = check_geometry(geom);
  if (rc) return rc;
  rc = check_pool(pool);
  if (rc) return rc;
  if (n_pages < 0 || n_requests < 0) return BIKV_ERR_BAD_ARG;
  if (n_pages == 0) return BIKV_OK;
  if (!recs || !requests || n_requests == 0) return BIKV_ERR_BAD_ARG;
  const int64_t total_pages = pool->pages_per_shard * pool->n_shards;
  for (int32_t r = 0; r < n_requests; ++r) {
    if (requests[r].tokens < 0) return BIKV_ERR_BAD_ARG;
    if (requests[r].base && worker_base_status((unsigned long long)(uintptr_t)requests[r].base))
      return BIKV_ERR_ALIGNMENT;
  }
  for (int64_t i = 0; i < n_pages; ++i) {
    const bikv_page_rec& p = recs[i];
    if (p.page_id < 0 || p.page_id >= total_pages) return BIKV_ERR_PAGE_RANGE;
    if (p.valid_tokens < 1 || p.valid_tokens > geom->page_tokens) return BIKV_ERR_PLAN;
    if (p.request < 0 || p.request >= n_requests) return BIKV_ERR_BAD_ARG;
    if (p.token_offset < 0 || (int64_t)p.token_offset + p.valid_tokens > requests[p.request].tokens)
      return BIKV_ERR_DST_RANGE;
  }
  if (check_overlap) {
    if (total_pages <= (int64_t)1 << 26) {
      // One bit per pool page (8 MiB at most), kept per thread between calls and
      // cleared again bit by bit, so the check is O(n_pages).
      thread_local std::vector<uint64_t> seen;
      const size_t words = (size_t)((total_pages + 63) / 64);
      if (seen.size() < words) seen.assign(words, 0);
      bool dup = false;
      int64_t done = 0;
      for (; done < n_pages && !dup; ++done) {
        const uint32_t id = (uint32_t)recs[done].page_id;
        uint64_t& wd = seen[id >> 6];
        const uint64_t bit = 1ull << (id & 63);
        dup = (wd & bit) != 0;
        wd |= bit;
      }
      for (int64_t i = 0; i < done; ++i) seen[(uint32_t)recs[i].page_id >> 6] = 0;
      if (dup) return BIKV_ERR_OVERLAP;
    } else {
      std::vector<int32_t> ids((size_t)n_pages);
      for (int64_t i = 0; i < n_pages; ++i) ids[(size_t)i] = recs[i].page_id;
      std::sort(ids.begin(), ids.end());
      if (std::adjacent_find(ids.begin(), ids.end()) != ids.end()) return BIKV_ERR_OVERLAP;
    }
  }
  return BIKV_OK;
}

static int run_nhd(const bikv_pool_desc* pool, const bikv_geometry* geom, const bikv_page_rec* recs_dev,
                   int64_t n_pages, void* const* layer_bases_dev, int64_t slots_per_layer, int to_pool,
                   int32_t* status_dev, void* stream) {
  int rc = check_geometry(geom);
  if (rc) return rc;
  rc = check_pool(pool);
  if (rc) return rc;
  if (geom->pool_layout != BIKV_POOL_PAGED || n_pages < 0 || slots_per_layer < 0) return BIKV_ERR_BAD_ARG;
  if (n_pages == 0) return BIKV_OK;
  if (!recs_dev || !layer_bases_dev) return BIKV_ERR_BAD_ARG;
  DeviceInfo di;
  rc = device_info(&di);
  if (rc) return rc;
  NhdArgs a;
  memset(&a, 0, sizeof(a));
  a.recs = reinterpret_cast<const uint4*>(recs_dev);
  a.layer_bases = reinterpret_cast<char* const*>(layer_bases_dev);
  a.pool = to_dev(pool);
  a.planes = 2u * geom->n_layers;
  a.row_bytes = (unsigned)(geom->n_kv_heads * geom->head_dim * geom->elt_bytes);
  // 32-byte accesses when the knob allows and rows are 32-byte multiples (the layer bases are
  // checked for that alignment in the kernel); U accesses in flight per lane either way.
  const bool wide = g_ldst_wide.load() != 0 && a.row_bytes % 32 == 0;
  a.row_vecs = a.row_bytes / (wide ? 32 : 16);
  a.row_vecs_m = a.row_vecs == 1 ? 0u : (unsigned)((1ull << 32) / a.row_vecs + 1);
  a.plane_bytes = a.row_bytes * geom->page_tokens;
  a.page_bytes = (unsigned long long)a.plane_bytes * a.planes;
  const long long items = n_pages * (long long)a.planes;
  if (items > 0x7fffffffll) return BIKV_ERR_TOO_LARGE;
  a.n_items = (unsigned)items;
  a.to_pool = to_pool;
  a.status = status_dev;
  a.page_tokens = (unsigned)geom->page_tokens;
  a.total_pages = (unsigned long long)pool->pages_per_shard * pool->n_shards;
  a.slots_per_layer = slots_per_layer;
  const int threads = 256, warps = threads / 32;
  const long long want = (items + warps - 1) / warps;
  const unsigned grid = (unsigned)std::min<long long>(want, (long long)di.sm_count * g_ldst_ctas_per_sm.load());
  if (wide)
    k_paged_nhd<4, 32><<<grid, threads, 0, (cudaStream_t)stream>>>(a);
  else
    k_paged_nhd<8, 16><<<grid, threads, 0, (cudaStream_t)stream>>>(a);
  return after_launch();
}

int bikv_gather_nhd(const bikv_pool_desc* pool, const bikv_geometry* geom, const bikv_page_rec* recs_dev,
                    int64_t n_pages, void* const* layer_bases_dev, int64_t slots_per_layer,
                    int32_t* status_dev, void* stream) {
  return run_nhd(pool, geom, recs_dev, n_pages, layer_bases_dev, slots_per_layer, 0, status_dev, stream);
}

int bikv_scatter_nhd(const bikv_pool_desc* pool, const bikv_geometry* geom, const bikv_page_rec* recs_dev,
                     int64_t n_pages, void* const* layer_bases_dev, int64_t slots_per_layer,
                     int32_t* status_dev, void* stream) {
  return run_nhd(pool, geom, recs_dev, n_pages, layer_bases_dev, slots_per_layer, 1, status_dev, stream);
}

int bikv_plan_validate_nhd(const bikv_page_rec* recs, int64_t n_pages, int64_t slots_per_layer,
                           const bikv_pool_desc* pool, const bikv_geometry* geom, int check_overlap) {
  if (slots_per_layer < 0) return BIKV_ERR_BAD_ARG;
  // Same checks as for contiguous worker tensors, with one window of slots_per_layer
  // tokens that every record must fall into.
  if (n_pages > 0 && !recs) return BIKV_ERR_BAD_ARG;
  for (int64_t i = 0; i < n_pages; ++i)
    if (recs[i].token_offset < 0 || (int64_t)recs[i].token_offset + recs[i].valid_tokens > slots_per_layer)
      return BIKV_ERR_DST_RANGE;
  std::vector<bikv_page_rec> tmp(recs, recs + n_pages);
  for (auto& r : tmp) r.request = 0;
  bikv_request_desc window{nullptr, slots_per_layer};
  return bikv_plan_validate(tmp.data(), n_pages, &window, 1, pool, geom, check_overlap);
}

int bikv_gather(const bikv_pool_desc* pool, const bikv_geometry* geom, const bikv_page_rec* recs_dev,
                int64_t n_pages, const bikv_request_desc* requests_dev, int32_t n_requests,
                int variant, int32_t* status_dev, void* stream) {
  return run(pool, geom, recs_dev, n_pages, requests_dev, n_requests, 0, variant, status_dev, stream);
}

int bikv_scatter(const bikv_pool_desc* pool, const bikv_geometry* geom, const bikv_page_rec* recs_dev,
                 int64_t n_pages, const bikv_request_desc* requests_dev, int32_t n_requests,
                 int variant, int32_t* status_dev, void* stream) {
  return run(pool, geom, recs_dev, n_pages, requests_dev, n_requests, 1, variant, status_dev, stream);
}

int64_t bikv_plan_scratch_bytes(int64_t n_pages, int32_t n_requests) {
  if (n_pages < 0 || n_requests < 0) return BIKV_ERR_BAD_ARG;
  const int64_t rec = ((int64_t)n_pages * (int64_t)sizeof(bikv_page_rec) + 255) & ~(int64_t)255;
  const int64_t req = ((int64_t)n_requests * (int64_t)sizeof(bikv_request_desc) + 255) & ~(int64_t)255;
  return rec + req;
}

int bikv_gather_h(const bikv_pool_desc* pool, const bikv_geometry* geom, const bikv_page_rec* recs_host,
                  int64_t n_pages, const bikv_request_desc* requests_host, int32_t n_requests,
                  void* plan_scratch_dev, int64_t plan_scratch_bytes, int validate, int variant,
                  int32_t* status_dev, void* stream) {
  return run_h(pool, geom, recs_host, n_pages, requests_host, n_requests, plan_scratch_dev,
               plan_scratch_bytes, validate, 0, variant, status_dev, stream);
}

int bikv_scatter_h(const bikv_pool_desc* pool, const bikv_geometry* geom, const bikv_page_rec* recs_host,
                   int64_t n_pages, const bikv_request_desc* requests_host, int32_t n_requests,
                   void* plan_scratch_dev, int64_t plan_scratch_bytes, int validate, int variant,
                   int32_t* status_dev, void* stream) {
  return run_h(pool, geom, recs_host, n_pages, requests_host, n_requests, plan_scratch_dev,
               plan_scratch_bytes, validate, 1, variant, status_dev, stream);
}

int bikv_copy_pages_flat(const void* src, void* dst, const int64_t* src_off_dev,
                         const int64_t* dst_off_dev, int64_t n_pages, int64_t page_elems,
                         int32_t elt_bytes, void* stream) {
  if (n_pages < 0 || page_elems < 0 || elt_bytes <= 0 || elt_bytes > 16) return BIKV_ERR_BAD_ARG;
  if (n_pages == 0 || page_elems == 0) return BIKV_OK;
  if (!src || !dst) return BIKV_ERR_BAD_ARG;
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc) return rc;
  FlatArgs a;
  memset(&a, 0, sizeof(a));
  a.src = (const char*)src;
  a.dst = (char*)dst;
  a.src_off = (const long long*)src_off_dev;
  a.dst_off = (const long long*)dst_off_dev;
  a.page_bytes = (unsigned long long)page_elems * elt_bytes;
  a.seg_bytes = (unsigned)g_ldst_seg_bytes.load();
  const unsigned long long parts = (a.page_bytes + a.seg_bytes - 1) / a.seg_bytes;
  if (parts > 0x7fffffffull) return BIKV_ERR_TOO_LARGE;
  a.parts = (unsigned)parts;
  a.n_items = (unsigned long long)n_pages * parts;
  a.elt_bytes = (unsigned)elt_bytes;
  a.wide = (int)g_ldst_wide.load();
  const int threads = 256, warps = threads / 32;
  const unsigned long long want = (a.n_items + warps - 1) / warps;
  unsigned grid = (unsigned)std::min<unsigned long long>(
      want, (unsigned long long)di.sm_count * g_ldst_ctas_per_sm.load());
  k_flat<8><<<grid, threads, 0, (cudaStream_t)stream>>>(a);
  return after_launch();
}

int bikv_selftest_wait_timeout(int32_t* status_dev, int64_t limit_ns, void* stream) {
  if (!status_dev || limit_ns <= 0 || limit_ns > 1000000000ll) return BIKV_ERR_BAD_ARG;
  k_selftest_wait_timeout<<<1, 32, 0, (cudaStream_t)stream>>>(status_dev, (unsigned long long)limit_ns);
  return after_launch();
}

int bikv_copy_range(void* dst, const void* src, int64_t bytes, void* stream) {
  if (bytes < 0) return BIKV_ERR_BAD_ARG;
  return bikv_copy_pages_flat(src, dst, nullptr, nullptr, 1, bytes, 1, stream);
}

int bikv_copy_range_engine(void* dst, const void* src, int64_t bytes, void* stream) {
  if (bytes < 0) return BIKV_ERR_BAD_ARG;
  if (bytes == 0) return BIKV_OK;
  if (!dst || !src) return BIKV_ERR_BAD_ARG;
  BIKV_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, (cudaStream_t)stream));
  return BIKV_OK;
}

int bikv_host_register(void* ptr, int64_t bytes) {
  if (!ptr || bytes <= 0) return BIKV_ERR_BAD_ARG;
  BIKV_CUDA(cudaHostRegister(ptr, (size_t)bytes, cudaHostRegisterPortable | cudaHostRegisterMapped));
  return BIKV_OK;
}

int bikv_host_unregister(void* ptr) {
  if (!ptr) return BIKV_ERR_BAD_ARG;
  BIKV_CUDA(cudaHostUnregister(ptr));
  return BIKV_OK;
}

int bikv_can_access_peer(int device, int peer, int* can) {
  if (!can) return BIKV_ERR_BAD_ARG;
  if (device == peer) {
    *can = 1;
    return BIKV_OK;
  }
  BIKV_CUDA(cudaDeviceCanAccessPeer(can, device, peer));
  return BIKV_OK;
}

int bikv_enable_peer(int device, int peer) {
  if (device == peer) return BIKV_OK;
  int can = 0;
  BIKV_CUDA(cudaDeviceCanAccessPeer(&can, device, peer));
  if (!can) return BIKV_ERR_PEER;
  int prev = 0;
  BIKV_CUDA(cudaGetDevice(&prev));
  BIKV_CUDA(cudaSetDevice(device));
  cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();
    e = cudaSuccess;
  }
  cudaError_t e2 = cudaSetDevice(prev);
  if (e != cudaSuccess) {
    cuda_fail(e);
    return BIKV_ERR_PEER;
  }
  BIKV_CUDA(e2);
  return BIKV_OK;
}

int bikv_pool_export(void* ptr, unsigned char handle[64], int64_t* offset) {
  if (!ptr || !handle || !offset) return BIKV_ERR_BAD_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handle is 64 bytes");
  // The handle names the whole allocation; find its base through the driver
  // entry point (no link-time dependency on libcuda).
  typedef int (*get_range_fn)(unsigned long long*, size_t*, unsigned long long);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  BIKV_CUDA(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres));
  if (!fn || qres != cudaDriverEntryPointSuccess) return BIKV_ERR_PEER;
  unsigned long long base = 0;
  size_t size = 0;
  if (((get_range_fn)fn)(&base, &size, (unsigned long long)(uintptr_t)ptr) != 0) return BIKV_ERR_PEER;
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, (void*)(uintptr_t)base);
  if (e != cudaSuccess) {
    cuda_fail(e);
    return BIKV_ERR_PEER;
  }
  memcpy(handle, &h, 64);
  *offset = (int64_t)((unsigned long long)(uintptr_t)ptr - base);
  return BIKV_OK;
}

int bikv_pool_import(const unsigned char handle[64], int64_t offset, void** ptr) {
  if (!handle || !ptr || offset < 0) return BIKV_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* base = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cuda_fail(e);
    return BIKV_ERR_PEER;
  }
  *ptr = (char*)base + offset;
  return BIKV_OK;
}

int bikv_pool_close(void* ptr, int64_t offset) {
  if (!ptr || offset < 0) return BIKV_ERR_BAD_ARG;
  // cudaIpcCloseMemHandle wants the base address that cudaIpcOpenMemHandle returned.
  cudaError_t e = cudaIpcCloseMemHandle((char*)ptr - offset);
  if (e != cudaSuccess) {
    cuda_fail(e);
    return BIKV_ERR_PEER;
  }
  return BIKV_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// bikv_gather_h_static: the gather for callers that cannot allocate.
//
// The plan staging area is this file-scope device array instead of a buffer the
// caller (or anyone) allocates.  In host code the name `g_static_plan` is only
// a stand-in for the symbol, not a device address: the address a kernel or a
// copy may use comes from cudaGetSymbolAddress, looked up once per device with
// that device current and cached below.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_plan[BIKV_STATIC_PLAN_BYTES];

namespace {
std::mutex g_static_mu;
void* g_static_addr[64] = {nullptr};

// Device address of g_static_plan on the current device (set-up on first use).
int static_plan_address(unsigned char** out) {
  int dev = 0;
  BIKV_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return BIKV_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_addr[dev]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_static_plan);
    if (e != cudaSuccess) return cuda_fail(e);
    if (!ptr) return BIKV_ERR_CUDA;
    g_static_addr[dev] = ptr;
  }
  *out = (unsigned char*)g_static_addr[dev];
  return BIKV_OK;
}
}  // namespace

extern "C" int bikv_gather_h_static(const bikv_pool_desc* pool, const bikv_geometry* geom,
                                    const bikv_page_rec* recs_host, int64_t n_pages,
                                    const bikv_request_desc* requests_host, int32_t n_requests,
                                    int validate, int variant, int32_t* status_dev, void* stream) {
  if (n_pages < 0 || n_requests < 0) return BIKV_ERR_BAD_ARG;
  if (n_pages > BIKV_STATIC_MAX_PAGES || n_requests > BIKV_STATIC_MAX_REQUESTS) return BIKV_ERR_TOO_LARGE;
  // Looked up before the empty-plan return, so that a call with n_pages == 0 serves as the
  // start-up call that places the array on the device.
  unsigned char* scratch = nullptr;
  int rc = static_plan_address(&scratch);
  if (rc) return rc;
  if (n_pages == 0) return BIKV_OK;
  if (!recs_host || !requests_host || n_requests == 0) return BIKV_ERR_BAD_ARG;
  for (int32_t r = 0; r < n_requests; ++r)
    if (!requests_host[r].base) return BIKV_ERR_BAD_ARG;
  if (validate) {
    rc = bikv_plan_validate(recs_host, n_pages, requests_host, n_requests, pool, geom, 0);
    if (rc) return rc;
  }
  // Records at the front, request table behind the record area's full extent.
  unsigned char* d_recs = scratch;
  unsigned char* d_reqs = scratch + (size_t)BIKV_STATIC_MAX_PAGES * sizeof(bikv_page_rec);
  cudaStream_t st = (cudaStream_t)stream;
  BIKV_CUDA(cudaMemcpyAsync(d_recs, recs_host, (size_t)n_pages * sizeof(bikv_page_rec),
                            cudaMemcpyHostToDevice, st));
  BIKV_CUDA(cudaMemcpyAsync(d_reqs, requests_host, (size_t)n_requests * sizeof(bikv_request_desc),
                            cudaMemcpyHostToDevice, st));
  return run(pool, geom, (const bikv_page_rec*)d_recs, n_pages, (const bikv_request_desc*)d_reqs,
             n_requests, 0, variant, status_dev, stream);
}
