// Device code of the KV-page data path: pure data movement, no arithmetic.
//
// Paged pool (page = [layer][kv][token][head][dim]):
//   k_paged_ldst      one warp per (page, plane, part) chunk, 16-byte ld/st
//   k_paged_bulk      one issuing thread per CTA, cp.async.bulk ring
//                     global -> shared -> global (no tensor map; plain, CTA-local
//                     bulk copies only)
//   k_paged_nhd       same chunks against a worker whose KV is paged per layer
//                     ([slot][kv][head][dim])
// Token-major pool of the reference (token = [dim][head][layer][kv]):
//   k_token_major16v  2-byte elements: swizzled 16-byte shared-memory units,
//                     cp.async double buffering of the pool rows (gather) or of
//                     the worker vectors (scatter)
//   k_token_major16   2-byte elements, any layer count: 4-byte units, odd pitch
//   k_token_major<T>  1- and 4-byte elements
// Flat reference copy:
//   k_flat            dst[dst_off[i]+e] = src[src_off[i]+e], any alignment
//
// A "plane" is one (layer, kv) pair; in the paged layout a page holds
// 2*n_layers planes of page_tokens*heads*dim elements each, so a plane of a
// page and its window in the worker tensor are both contiguous byte runs.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "bikv.h"

namespace bikv {

struct PoolDev {
  char* base[BIKV_MAX_SHARDS];
  int n_shards;
  int rule;
  long long pages_per_shard;
};

struct PagedArgs {
  const uint4* recs;               // bikv_page_rec viewed as 16-byte words
  const bikv_request_desc* reqs;
  PoolDev pool;
  unsigned n_items;                // n_pages * planes * parts
  unsigned planes;                 // 2 * n_layers
  unsigned parts;                  // ceil(plane_bytes / seg_bytes)
  unsigned seg_bytes;
  unsigned row_bytes;              // heads * dim * elt_bytes (one token of one plane)
  unsigned plane_bytes;            // page_tokens * row_bytes
  unsigned long long page_bytes;   // planes * plane_bytes
  int to_pool;                     // 0 = gather (pool -> worker), 1 = scatter
  int* status;
  unsigned n_requests;             // bounds for the record checks below
  unsigned page_tokens;
  unsigned long long total_pages;  // n_shards * pages_per_shard
  int wide;                        // ld/st kernel: 32-byte accesses where both sides are 32-byte aligned
  unsigned span;                   // bulk ring: adjacent planes per item (1 = one plane or part)
  unsigned groups;                 // ceil(planes / span)
};

// A record that points outside the pool or outside its worker tensor is skipped, never
// dereferenced, and the first such error is left in the caller's status word (if one was
// given): plans that reach the device entry points cannot be checked on the host.
__device__ __forceinline__ bool record_ok(const uint4& r, unsigned n_requests, unsigned page_tokens,
                                          unsigned long long total_pages, int* status) {
#ifdef BIKV_NO_RECORD_CHECKS   // measurement builds only
  return true;
#endif
  int err = 0;
  if ((unsigned long long)r.x >= total_pages)
    err = BIKV_ERR_PAGE_RANGE;
  else if (r.y == 0 || r.y > page_tokens)
    err = BIKV_ERR_PLAN;
  else if (r.z >= n_requests)
    err = BIKV_ERR_BAD_ARG;
  else if ((int)r.w < 0)
    err = BIKV_ERR_DST_RANGE;
  if (err == 0) return true;
  if (status) atomicCAS(status, 0, err);
  return false;
}
// The one rule for a worker-side base address (a request's KV tensor, a layer tensor of a
// paged worker cache): not null and 16-byte aligned, because bulk copies, cp.async and the
// vector loads and stores are issued on addresses derived from it.  Host validation and
// every kernel use this same function.
__host__ __device__ __forceinline__ int worker_base_status(unsigned long long base) {
  if (base == 0) return BIKV_ERR_BAD_ARG;
  if (base & 15ull) return BIKV_ERR_ALIGNMENT;
  return BIKV_OK;
}
// Checks the request descriptor a record selected: its base address and that the record's
// token window lies inside the tensor.  Called before any address is formed from `base`.
__device__ __forceinline__ bool window_ok(const uint4& r, unsigned long long base, long long tensor_tokens,
                                          int* status) {
#ifdef BIKV_NO_RECORD_CHECKS
  return true;
#endif
  int err = worker_base_status(base);
  if (err == 0 && (long long)r.w + (long long)r.y > tensor_tokens) err = BIKV_ERR_DST_RANGE;
  if (err == 0) return true;
  if (status) atomicCAS(status, 0, err);
  return false;
}

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream16(void* p, const uint4& v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

struct Vec32 {
  unsigned r[8];
};
__device__ __forceinline__ Vec32 ld_stream32(const void* p) {
  Vec32 v;
  asm volatile("ld.global.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.r[0]), "=r"(v.r[1]), "=r"(v.r[2]), "=r"(v.r[3]), "=r"(v.r[4]), "=r"(v.r[5]), "=r"(v.r[6]),
                 "=r"(v.r[7])
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream32(void* p, const Vec32& v) {
  asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.r[0]),
               "r"(v.r[1]), "r"(v.r[2]), "r"(v.r[3]), "r"(v.r[4]), "r"(v.r[5]), "r"(v.r[6]), "r"(v.r[7])
               : "memory");
}

// Resolves chunk w to (pool address, worker address, byte count).  Returns
// false for a part that lies wholly beyond the valid tokens of a partial page.
__device__ __forceinline__ bool decode_item(const PagedArgs& a, unsigned w, char*& pool_p,
                                            char*& work_p, unsigned& bytes) {
  const unsigned part = w % a.parts;
  const unsigned t = w / a.parts;
  const unsigned plane = t % a.planes;
  const unsigned page = t / a.planes;
  const uint4 r = __ldg(a.recs + page);
  if (!record_ok(r, a.n_requests, a.page_tokens, a.total_pages, a.status)) return false;
  const unsigned vbytes = r.y * a.row_bytes;
  const unsigned off = part * a.seg_bytes;
  if (off >= vbytes) return false;
  bytes = min(a.seg_bytes, vbytes - off);
  const unsigned id = r.x;
  unsigned shard;
  unsigned long long local;
  if (a.pool.rule == BIKV_SHARD_MOD) {
    shard = id % (unsigned)a.pool.n_shards;
    local = id / (unsigned)a.pool.n_shards;
  } else {
    shard = (unsigned)(id / a.pool.pages_per_shard);
    local = id % a.pool.pages_per_shard;
  }
  pool_p = a.pool.base[shard] + local * a.page_bytes + (unsigned long long)plane * a.plane_bytes + off;
  const longlong2 rq = __ldg(reinterpret_cast<const longlong2*>(a.reqs + r.z));
  if (!window_ok(r, (unsigned long long)rq.x, rq.y, a.status)) return false;
  work_p = reinterpret_cast<char*>(rq.x) +
           ((unsigned long long)plane * (unsigned long long)rq.y + r.w) * a.row_bytes + off;
  return true;
}

// Both addresses 16-byte aligned: 16-byte accesses, U in flight per lane; with `wide` and
// 32-byte alignment the bulk goes in 32-byte accesses (a warp instruction then covers 1 KiB).
template <int U>
__device__ __forceinline__ void warp_copy_aligned(const char* src, char* dst, unsigned long long bytes, int lane,
                                                  bool wide) {
  if (wide && (((unsigned long long)src | (unsigned long long)dst) & 31) == 0 && bytes >= 1024) {
    constexpr int W = U / 2;
    const unsigned long long n = bytes >> 5;
    unsigned long long i = lane;
    for (; i + 32ull * (W - 1) < n; i += 32ull * W) {
      Vec32 v[W];
#pragma unroll
      for (int u = 0; u < W; ++u) v[u] = ld_stream32(src + ((i + 32 * u) << 5));
#pragma unroll
      for (int u = 0; u < W; ++u) st_stream32(dst + ((i + 32 * u) << 5), v[u]);
    }
    for (; i < n; i += 32) st_stream32(dst + (i << 5), ld_stream32(src + (i << 5)));
    src += n << 5;
    dst += n << 5;
    bytes -= n << 5;
  }
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  const unsigned long long n = bytes >> 4;
  unsigned long long i = lane;
  for (; i + 32ull * (U - 1) < n; i += 32ull * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = ld_stream16(s + i + 32 * u);
#pragma unroll
    for (int u = 0; u < U; ++u) st_stream16(d + i + 32 * u, v[u]);
  }
  for (; i < n; i += 32) st_stream16(d + i, ld_stream16(s + i));
  for (unsigned long long b = (n << 4) + lane; b < bytes; b += 32) dst[b] = src[b];
}

// Copies `bytes` from src to dst with the 32 lanes of one warp.  Fast path:
// both 16-byte aligned.  Otherwise the widest power-of-two unit that divides
// both addresses is used, with a byte tail.
template <int U>
__device__ __forceinline__ void warp_copy(const char* src, char* dst, unsigned long long bytes,
                                          int lane, bool wide = false) {
  const unsigned long long mis = (unsigned long long)src | (unsigned long long)dst;
  if ((mis & 15) == 0) {
    warp_copy_aligned<U>(src, dst, bytes, lane, wide);
    return;
  }
  if (((unsigned long long)src & 15) == ((unsigned long long)dst & 15)) {
    // Same misalignment on both sides: peel a byte head, then the aligned path.
    unsigned long long head = 16 - ((unsigned long long)src & 15);
    if (head > bytes) head = bytes;
    for (unsigned long long b = lane; b < head; b += 32) dst[b] = src[b];
    if (bytes > head) warp_copy_aligned<U>(src + head, dst + head, bytes - head, lane, wide);
    return;
  }
  if ((mis & 7) == 0) {
    const unsigned long long n = bytes >> 3;
    for (unsigned long long i = lane; i < n; i += 32)
      reinterpret_cast<unsigned long long*>(dst)[i] = reinterpret_cast<const unsigned long long*>(src)[i];
    for (unsigned long long b = (n << 3) + lane; b < bytes; b += 32) dst[b] = src[b];
  } else if ((mis & 3) == 0) {
    const unsigned long long n = bytes >> 2;
    for (unsigned long long i = lane; i < n; i += 32)
      reinterpret_cast<unsigned*>(dst)[i] = reinterpret_cast<const unsigned*>(src)[i];
    for (unsigned long long b = (n << 2) + lane; b < bytes; b += 32) dst[b] = src[b];
  } else if ((mis & 1) == 0) {
    const unsigned long long n = bytes >> 1;
    for (unsigned long long i = lane; i < n; i += 32)
      reinterpret_cast<unsigned short*>(dst)[i] = reinterpret_cast<const unsigned short*>(src)[i];
    for (unsigned long long b = (n << 1) + lane; b < bytes; b += 32) dst[b] = src[b];
  } else {
    for (unsigned long long b = lane; b < bytes; b += 32) dst[b] = src[b];
  }
}

// ---------------------------------------------------------------------------
// Paged layout, direct ld/st.  Adjacent warps take adjacent planes of a page,
// so a CTA reads one contiguous stretch of the pool page per sweep.
// ---------------------------------------------------------------------------
template <int U>
__global__ void __launch_bounds__(256) k_paged_ldst(const __grid_constant__ PagedArgs a) {
  const int lane = threadIdx.x & 31;
  const unsigned warps_per_cta = blockDim.x >> 5;
  const unsigned stride = gridDim.x * warps_per_cta;
  for (unsigned w = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); w < a.n_items; w += stride) {
    char *pool_p, *work_p;
    unsigned bytes;
    if (!decode_item(a, w, pool_p, work_p, bytes)) continue;
    if (a.to_pool)
      warp_copy<U>(work_p, pool_p, bytes, lane, a.wide != 0);
    else
      warp_copy<U>(pool_p, work_p, bytes, lane, a.wide != 0);
  }
}

// ---------------------------------------------------------------------------
// Paged pool <-> paged worker KV ([slot][kv][head][dim] per layer).  One warp per
// (page, plane): the plane of the page is one contiguous run of valid_tokens rows;
// on the worker side row t lies 2 rows further than row t-1 (K and V rows of a
// slot alternate).
// ---------------------------------------------------------------------------
struct NhdArgs {
  const uint4* recs;
  char* const* layer_bases;
  PoolDev pool;
  unsigned n_items;        // n_pages * planes
  unsigned planes;
  unsigned row_bytes;
  unsigned row_vecs;       // row_bytes / bytes per access (16 or 32)
  unsigned row_vecs_m;     // multiply-high constant for division by row_vecs (0 when 1)
  unsigned plane_bytes;
  unsigned long long page_bytes;
  int to_pool;
  int* status;
  unsigned page_tokens;
  unsigned long long total_pages;
  long long slots_per_layer;
};

// VB = bytes per access: 16, or 32 when rows and bases are 32-byte aligned.
template <int VB>
struct NhdVec;
template <>
struct NhdVec<16> {
  using T = uint4;
  static __device__ __forceinline__ T ld(const char* p) { return ld_stream16(p); }
  static __device__ __forceinline__ void st(char* p, const T& v) { st_stream16(p, v); }
};
template <>
struct NhdVec<32> {
  using T = Vec32;
  static __device__ __forceinline__ T ld(const char* p) { return ld_stream32(p); }
  static __device__ __forceinline__ void st(char* p, const T& v) { st_stream32(p, v); }
};

template <int U, int VB>
__global__ void __launch_bounds__(256) k_paged_nhd(const __grid_constant__ NhdArgs a) {
  using V = NhdVec<VB>;
  const unsigned lane = threadIdx.x & 31;
  const unsigned warps_per_cta = blockDim.x >> 5;
  const unsigned stride = gridDim.x * warps_per_cta;
  for (unsigned w = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); w < a.n_items; w += stride) {
    const unsigned plane = w % a.planes;
    const unsigned page = w / a.planes;
    uint4 r = __ldg(a.recs + page);
    r.z = 0;  // the request field is unused for a paged worker cache
    // The layer table lives in device memory like the records: its entry is checked (not
    // null, 16-byte aligned) together with the slot window, before any address is formed.
    const unsigned long long layer_addr = __ldg(reinterpret_cast<const unsigned long long*>(a.layer_bases) + (plane >> 1));
    if (!record_ok(r, 1, a.page_tokens, a.total_pages, a.status) ||
        !window_ok(r, layer_addr, a.slots_per_layer, a.status))
      continue;
    const unsigned id = r.x;
    unsigned shard;
    unsigned long long local;
    if (a.pool.rule == BIKV_SHARD_MOD) {
      shard = id % (unsigned)a.pool.n_shards;
      local = id / (unsigned)a.pool.n_shards;
    } else {
      shard = (unsigned)(id / a.pool.pages_per_shard);
      local = id % a.pool.pages_per_shard;
    }
    char* pool_p = a.pool.base[shard] + local * a.page_bytes + (unsigned long long)plane * a.plane_bytes;
    const unsigned kv = plane & 1;
    char* work_p = reinterpret_cast<char*>(layer_addr) + ((unsigned long long)r.w * 2 + kv) * a.row_bytes;
    if (VB == 32 && (layer_addr & 31)) {
      // A layer tensor aligned to 16 but not to 32 bytes in a launch sized for 32-byte accesses:
      // this plane goes in 16-byte accesses (rare; not worth a tuned loop).
      const unsigned rv = a.row_vecs * 2, n16 = r.y * rv;
      for (unsigned i = lane; i < n16; i += 32) {
        const unsigned long long wofs = (unsigned long long)(i + (i / rv) * rv) * 16;
        if (!a.to_pool)
          st_stream16(work_p + wofs, ld_stream16(pool_p + (unsigned long long)i * 16));
        else
          st_stream16(pool_p + (unsigned long long)i * 16, ld_stream16(work_p + wofs));
      }
      continue;
    }
    const unsigned n = r.y * a.row_vecs;          // accesses of VB bytes in the valid rows
    auto wo = [&](unsigned i) -> unsigned long long {   // worker-side byte offset of pool-side access i
      const unsigned t = a.row_vecs_m ? __umulhi(i, a.row_vecs_m) : i;
      return (unsigned long long)(i + t * a.row_vecs) * VB;  // t*2*row_vecs + (i - t*row_vecs)
    };
    unsigned i = lane;
    if (!a.to_pool) {
      for (; i + 32u * (U - 1) < n; i += 32u * U) {
        typename V::T v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = V::ld(pool_p + (unsigned long long)(i + 32 * u) * VB);
#pragma unroll
        for (int u = 0; u < U; ++u) V::st(work_p + wo(i + 32 * u), v[u]);
      }
      for (; i < n; i += 32) V::st(work_p + wo(i), V::ld(pool_p + (unsigned long long)i * VB));
    } else {
      for (; i + 32u * (U - 1) < n; i += 32u * U) {
        typename V::T v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = V::ld(work_p + wo(i + 32 * u));
#pragma unroll
        for (int u = 0; u < U; ++u) V::st(pool_p + (unsigned long long)(i + 32 * u) * VB, v[u]);
      }
      for (; i < n; i += 32) V::st(pool_p + (unsigned long long)i * VB, V::ld(work_p + wo(i)));
    }
  }
}

// ---------------------------------------------------------------------------
// Paged layout, bulk-async ring.  Thread 0 of each CTA runs a software
// pipeline over `stages` shared-memory buffers of seg_bytes each:
//   load(k+stages-1) in flight | wait full(k) | store(k) | refill stage of k-1
// Every wait on an mbarrier is bounded; on expiry the thread records
// BIKV_ERR_DEVICE_TIMEOUT in status[0], stops issuing, drains its stores and
// gives every outstanding load one more bounded wait before returning.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: at most `limit_ns` of wall time (2 s in the copy ring) and at most
// 2^24 polls.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  unsigned long long limit_ns = 2000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long deadline = global_timer_ns() + limit_ns;
  for (unsigned i = 0; i < (1u << 24); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63) == 63 && global_timer_ns() > deadline) break;
  }
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_1() {
  asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

constexpr int kMaxStages = 12;

// One stage of the bulk ring: `np` adjacent planes of one page (np = 1 with `vbytes` the size
// of a part of a plane when planes are split, or when span is 1).  Pool side: the planes
// are adjacent, plane_bytes apart; worker side: `work_stride` apart.
struct BulkItem {
  char* pool_p;
  char* work_p;
  unsigned long long work_stride;
  unsigned vbytes;   // valid bytes of each plane (or of the part)
  unsigned np;       // planes in this item; 0 = nothing to copy
};

// Resolves item w of a launch whose items are (page, group of `span` adjacent planes).
__device__ __forceinline__ BulkItem decode_span(const PagedArgs& a, unsigned w) {
  BulkItem it;
  it.np = 0;
  if (a.span <= 1) {
    unsigned bytes;
    if (!decode_item(a, w, it.pool_p, it.work_p, bytes)) return it;
    it.work_stride = 0;
    it.vbytes = bytes;
    it.np = 1;
    return it;
  }
  const unsigned group = w % a.groups;
  const unsigned page = w / a.groups;
  const uint4 r = __ldg(a.recs + page);
  if (!record_ok(r, a.n_requests, a.page_tokens, a.total_pages, a.status)) return it;
  const unsigned plane0 = group * a.span;
  const unsigned id = r.x;
  unsigned shard;
  unsigned long long local;
  if (a.pool.rule == BIKV_SHARD_MOD) {
    shard = id % (unsigned)a.pool.n_shards;
    local = id / (unsigned)a.pool.n_shards;
  } else {
    shard = (unsigned)(id / a.pool.pages_per_shard);
    local = id % a.pool.pages_per_shard;
  }
  const longlong2 rq = __ldg(reinterpret_cast<const longlong2*>(a.reqs + r.z));
  if (!window_ok(r, (unsigned long long)rq.x, rq.y, a.status)) return it;
  it.pool_p = a.pool.base[shard] + local * a.page_bytes + (unsigned long long)plane0 * a.plane_bytes;
  it.work_stride = (unsigned long long)rq.y * a.row_bytes;
  it.work_p = reinterpret_cast<char*>(rq.x) + plane0 * it.work_stride + (unsigned long long)r.w * a.row_bytes;
  it.vbytes = r.y * a.row_bytes;
  it.np = min(a.span, a.planes - plane0);
  return it;
}

__global__ void __launch_bounds__(32) k_paged_bulk(const __grid_constant__ PagedArgs a, int stages) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bars[kMaxStages];
  if (threadIdx.x != 0) return;

  for (int s = 0; s < stages; ++s) mbar_init(smem_u32(&bars[s]), 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");

  const uint32_t buf0 = smem_u32(smem);
  const unsigned stage_bytes = a.seg_bytes * (a.span ? a.span : 1u);
  const unsigned stride = gridDim.x;
  // Number of items this CTA owns: w = blockIdx.x + k*stride.
  const unsigned mine = (a.n_items > blockIdx.x) ? (a.n_items - blockIdx.x + stride - 1) / stride : 0;

  unsigned phase_bits = 0;      // bit s = parity to wait for on stage s
  unsigned loaded_bits = 0;     // bit s = a load is outstanding on stage s
  BulkItem st[kMaxStages];      // the item held in each stage
  bool failed = false;

  // Gather: the planes of a pool page are adjacent, so ONE bulk load brings all of the
  // item's planes (up to the valid rows of the last one); each plane then leaves with its
  // own bulk store into its window of the worker tensor.  Scatter: one bulk load per
  // plane window, all counted on the stage's barrier; a full page's planes leave with one
  // store, a partial page's with one store per plane.
  auto issue_load = [&](unsigned k) {
    const int s = k % stages;
    st[s].np = 0;
    if (k >= mine) return;
    st[s] = decode_span(a, blockIdx.x + k * stride);
    const BulkItem& it = st[s];
    if (it.np == 0) return;
    const uint32_t bar = smem_u32(&bars[s]);
    const uint32_t buf = buf0 + s * stage_bytes;
    if (!a.to_pool) {
      const unsigned bytes = (it.np - 1) * a.plane_bytes + it.vbytes;
      mbar_expect_tx(bar, bytes);
      bulk_g2s(buf, it.pool_p, bytes, bar);
    } else {
      mbar_expect_tx(bar, it.np * it.vbytes);
      for (unsigned p = 0; p < it.np; ++p)
        bulk_g2s(buf + p * a.plane_bytes, it.work_p + p * it.work_stride, it.vbytes, bar);
    }
    loaded_bits |= 1u << s;
  };

  for (unsigned k = 0; k + 1 < (unsigned)stages && k < mine; ++k) issue_load(k);

  for (unsigned k = 0; k < mine; ++k) {
    const int s = k % stages;
    const BulkItem& it = st[s];
    if (it.np != 0) {
      if (!mbar_wait_bounded(smem_u32(&bars[s]), (phase_bits >> s) & 1)) {
        failed = true;
        break;
      }
      phase_bits ^= 1u << s;
      loaded_bits &= ~(1u << s);
      const uint32_t buf = buf0 + s * stage_bytes;
      if (!a.to_pool) {
        for (unsigned p = 0; p < it.np; ++p)
          bulk_s2g(it.work_p + p * it.work_stride, buf + p * a.plane_bytes, it.vbytes);
      } else if (it.np == 1 || it.vbytes == a.plane_bytes) {
        bulk_s2g(it.pool_p, buf, (it.np - 1) * a.plane_bytes + it.vbytes);
      } else {
        for (unsigned p = 0; p < it.np; ++p)
          bulk_s2g(it.pool_p + (unsigned long long)p * a.plane_bytes, buf + p * a.plane_bytes, it.vbytes);
      }
    }
    bulk_commit();
    // The stores of item k-1 have finished reading their stage once at most one
    // group (the one just committed) is still pending; that stage is the one
    // item k+stages-1 maps to.
    bulk_wait_read_1();
    issue_load(k + stages - 1);
  }

  bulk_wait_all();
  if (failed) {
    if (a.status) atomicExch(a.status, (int)BIKV_ERR_DEVICE_TIMEOUT);
    for (int s = 0; s < stages; ++s)
      if (loaded_bits & (1u << s)) (void)mbar_wait_bounded(smem_u32(&bars[s]), (phase_bits >> s) & 1);
  }
}

// Diagnostic: one thread waits, with a short limit, on an mbarrier whose transaction
// count nothing will ever satisfy, and reports the expiry exactly as the copy ring
// does.  Exercises the bounded wait and the status word without a fault or a hang.
__global__ void k_selftest_wait_timeout(int* status, unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar;
  if (threadIdx.x != 0) return;
  mbar_init(smem_u32(&bar), 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  mbar_expect_tx(smem_u32(&bar), 16);   // 16 bytes that no copy delivers
  if (!mbar_wait_bounded(smem_u32(&bar), 0, limit_ns)) atomicExch(status, (int)BIKV_ERR_DEVICE_TIMEOUT);
}

// ---------------------------------------------------------------------------
// Flat page copy (reference kernel semantics).  One warp per (page, part).
// ---------------------------------------------------------------------------
struct FlatArgs {
  const char* src;
  char* dst;
  const long long* src_off;  // elements; may be null (all zero)
  const long long* dst_off;
  unsigned long long page_bytes;
  unsigned long long n_items;  // n_pages * parts
  unsigned parts;
  unsigned seg_bytes;
  unsigned elt_bytes;
  int wide;
};

template <int U>
__global__ void __launch_bounds__(256) k_flat(const __grid_constant__ FlatArgs a) {
  const int lane = threadIdx.x & 31;
  const unsigned warps_per_cta = blockDim.x >> 5;
  const unsigned long long stride = (unsigned long long)gridDim.x * warps_per_cta;
  for (unsigned long long w = (unsigned long long)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
       w < a.n_items; w += stride) {
    const unsigned part = (unsigned)(w % a.parts);
    const unsigned long long page = w / a.parts;
    const unsigned long long off = (unsigned long long)part * a.seg_bytes;
    unsigned long long bytes = a.page_bytes - off;
    if (bytes > a.seg_bytes) bytes = a.seg_bytes;
    const long long so = a.src_off ? __ldg(a.src_off + page) : 0;
    const long long dn = a.dst_off ? __ldg(a.dst_off + page) : 0;
    warp_copy<U>(a.src + so * (long long)a.elt_bytes + off, a.dst + dn * (long long)a.elt_bytes + off,
                 bytes, lane, a.wide != 0);
  }
}

// ---------------------------------------------------------------------------
// Token-major (reference) pool <-> layer-major worker KV.
//
// Pool token row: element (d, h, c) at ((d*H + h)*C + c), c = layer*2 + kv,
// C = 2*n_layers.  Worker: element (c, tok, h, d) at ((c*T + tok)*H + h)*D + d.
// A CTA stages a slab of DT consecutive d (all heads, all planes) of one token
// in shared memory: the pool side of the slab is one contiguous run and moves
// with 16-byte accesses; the worker side moves as 16-byte vectors of V = 16/elt
// consecutive d for a fixed (c, h).  Lanes vary c fastest so the element-wise
// shared-memory accesses of a warp fall on consecutive addresses.
// ---------------------------------------------------------------------------
struct TokenMajorArgs {
  const uint4* recs;
  const bikv_request_desc* reqs;
  PoolDev pool;
  unsigned n_items;       // n_pages * page_tokens * slabs
  unsigned page_tokens;
  unsigned slabs;         // D / DT
  unsigned DT;            // d per slab (multiple of V)
  unsigned H, D, C;
  unsigned long long token_bytes;  // D*H*C*elt
  int to_pool;
  int* status;
  unsigned n_requests;
  unsigned long long total_pages;
};

template <typename T>
__global__ void __launch_bounds__(256) k_token_major(const __grid_constant__ TokenMajorArgs a) {
  extern __shared__ __align__(16) unsigned char tm_smem[];
  T* tile = reinterpret_cast<T*>(tm_smem);
  constexpr unsigned V = 16 / sizeof(T);
  const unsigned slab_elems = a.DT * a.H * a.C;
  const unsigned slab_vec = slab_elems / V;       // slab bytes / 16
  const unsigned groups = a.DT / V;               // d-groups per slab
  const unsigned n_out = a.C * a.H * groups;      // 16-byte worker vectors per slab

  for (unsigned w = blockIdx.x; w < a.n_items; w += gridDim.x) {
    const unsigned slab = w % a.slabs;
    const unsigned t = w / a.slabs;
    const unsigned tok = t % a.page_tokens;
    const unsigned page = t / a.page_tokens;
    const uint4 r = __ldg(a.recs + page);
    if (!record_ok(r, a.n_requests, a.page_tokens, a.total_pages, a.status)) continue;  // uniform across the CTA
    if (tok >= r.y) continue;
    const unsigned id = r.x;
    unsigned shard;
    unsigned long long local;
    if (a.pool.rule == BIKV_SHARD_MOD) {
      shard = id % (unsigned)a.pool.n_shards;
      local = id / (unsigned)a.pool.n_shards;
    } else {
      shard = (unsigned)(id / a.pool.pages_per_shard);
      local = id % a.pool.pages_per_shard;
    }
    char* pool_p = a.pool.base[shard] + (local * a.page_tokens + tok) * a.token_bytes +
                   (unsigned long long)slab * slab_elems * sizeof(T);
    const longlong2 rq = __ldg(reinterpret_cast<const longlong2*>(a.reqs + r.z));
    if (!window_ok(r, (unsigned long long)rq.x, rq.y, a.status)) continue;
    T* work = reinterpret_cast<T*>(rq.x);
    const unsigned long long T_req = (unsigned long long)rq.y;
    const unsigned long long wtok = r.w + tok;
    const unsigned d_base = slab * a.DT;

    if (!a.to_pool) {
      const uint4* s = reinterpret_cast<const uint4*>(pool_p);
      uint4* d = reinterpret_cast<uint4*>(tile);
      for (unsigned i = threadIdx.x; i < slab_vec; i += blockDim.x) d[i] = ld_stream16(s + i);
      __syncthreads();
      for (unsigned o = threadIdx.x; o < n_out; o += blockDim.x) {
        const unsigned c = o % a.C;
        const unsigned q = o / a.C;
        const unsigned h = q % a.H;
        const unsigned g = q / a.H;
        union { uint4 v; T e[V]; } u;
#pragma unroll
        for (unsigned j = 0; j < V; ++j) u.e[j] = tile[((g * V + j) * a.H + h) * a.C + c];
        T* dst = work + ((c * T_req + wtok) * a.H + h) * a.D + d_base + g * V;
        st_stream16(dst, u.v);
      }
      __syncthreads();
    } else {
      for (unsigned o = threadIdx.x; o < n_out; o += blockDim.x) {
        const unsigned c = o % a.C;
        const unsigned q = o / a.C;
        const unsigned h = q % a.H;
        const unsigned g = q / a.H;
        union { uint4 v; T e[V]; } u;
        const T* src = work + ((c * T_req + wtok) * a.H + h) * a.D + d_base + g * V;
        u.v = ld_stream16(src);
#pragma unroll
        for (unsigned j = 0; j < V; ++j) tile[((g * V + j) * a.H + h) * a.C + c] = u.e[j];
      }
      __syncthreads();
      const uint4* s = reinterpret_cast<const uint4*>(tile);
      uint4* d = reinterpret_cast<uint4*>(pool_p);
      for (unsigned i = threadIdx.x; i < slab_vec; i += blockDim.x) st_stream16(d + i, s[i]);
      __syncthreads();
    }
  }
}


// ---------------------------------------------------------------------------
// Token-major pool, 2-byte elements (fp16 / bf16): the fast path.
//
// A (K,V) pair of one (d, h, layer) is one 32-bit word of the pool row, and the
// row of a token is [d][h][layer] words.  A CTA moves a slab of Gs groups of 8
// consecutive d (all heads, all layers) of one token.  In shared memory the slab
// is kept as [j = d%8][h][g = d/8][layer] with an ODD layer pitch, so that
//   * worker side: lane (h, g) reads/writes its 8 words (j = 0..7) at a stride of
//     one pitch between lanes -- no bank conflicts -- and a warp's 16-byte
//     vectors of K (and of V) form one contiguous run of the worker tensor;
//   * pool side: the slab is one contiguous run, moved in 16-byte units.
// ---------------------------------------------------------------------------
// Division by a runtime constant as one multiply-high: exact while n * d < 2^32
// (items, words and rows of a slab are far below that).
struct FastDiv {
  unsigned d, m;  // m = floor(2^32 / d) + 1, or 0 when d == 1
  __device__ __forceinline__ unsigned div(unsigned n) const { return d == 1 ? n : __umulhi(n, m); }
};

struct TokenMajor16Args {
  const uint4* recs;
  const bikv_request_desc* reqs;
  PoolDev pool;
  unsigned n_items;      // n_pages * page_tokens * slabs
  unsigned page_tokens;
  unsigned slabs;        // G / Gs
  unsigned Gs;           // d-groups (of 8) per slab
  unsigned H, D, L;
  unsigned Lp;           // odd pitch >= L, in words
  FastDiv div_L, div_H, div_HG, div_Gs, div_slabs, div_ptok;
  unsigned long long token_bytes;  // D*H*L*4
  int to_pool;
  int* status;
  unsigned n_requests;
  unsigned long long total_pages;
};

// Shared-memory word index of (d_local, h, l): layout [j = d%8][h][g = d/8][l].
__device__ __forceinline__ unsigned tm16_index(const TokenMajor16Args& a, unsigned d_local, unsigned h, unsigned l) {
  return (((d_local & 7) * a.H + h) * a.Gs + (d_local >> 3)) * a.Lp + l;
}

__global__ void __launch_bounds__(256) k_token_major16(const __grid_constant__ TokenMajor16Args a) {
  extern __shared__ __align__(16) unsigned tm16_tile[];
  unsigned* tile = tm16_tile;
  const unsigned HG = a.H * a.Gs;
  const unsigned slab_words = a.Gs * 8 * a.H * a.L;
  const unsigned slab_units = slab_words >> 2;
  const unsigned n_out = a.L * HG;
  const unsigned row_elems = a.H * a.D;
  const unsigned j_pitch = a.H * a.Gs * a.Lp;   // words between j and j+1

  for (unsigned w = blockIdx.x; w < a.n_items; w += gridDim.x) {
    const unsigned t = a.div_slabs.div(w);
    const unsigned slab = w - t * a.slabs;
    const unsigned page = a.div_ptok.div(t);
    const unsigned tok = t - page * a.page_tokens;
    const uint4 r = __ldg(a.recs + page);
    if (!record_ok(r, a.n_requests, a.page_tokens, a.total_pages, a.status)) continue;  // uniform across the CTA
    if (tok >= r.y) continue;
    const unsigned id = r.x;
    unsigned shard;
    unsigned long long local;
    if (a.pool.rule == BIKV_SHARD_MOD) {
      shard = id % (unsigned)a.pool.n_shards;
      local = id / (unsigned)a.pool.n_shards;
    } else {
      shard = (unsigned)(id / a.pool.pages_per_shard);
      local = id % a.pool.pages_per_shard;
    }
    uint4* pool_p = reinterpret_cast<uint4*>(a.pool.base[shard] + (local * a.page_tokens + tok) * a.token_bytes +
                                             (unsigned long long)slab * slab_words * 4ull);
    const longlong2 rq = __ldg(reinterpret_cast<const longlong2*>(a.reqs + r.z));
    if (!window_ok(r, (unsigned long long)rq.x, rq.y, a.status)) continue;
    unsigned short* work = reinterpret_cast<unsigned short*>(rq.x);
    const unsigned long long T_req = (unsigned long long)rq.y;
    // Element offset of (plane 0, this token, h = 0, first d of the slab); a plane is
    // T_req * row_elems elements further.
    unsigned short* work_tok = work + (unsigned long long)(r.w + tok) * row_elems + slab * a.Gs * 8;
    const unsigned long long plane_elems = T_req * row_elems;

    if (!a.to_pool) {
      // pool -> shared (16-byte units of the contiguous slab)
      for (unsigned i0 = threadIdx.x; i0 < slab_units; i0 += 4 * blockDim.x) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const unsigned i = i0 + u * blockDim.x;
          if (i < slab_units) v[u] = ld_stream16(pool_p + i);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const unsigned i = i0 + u * blockDim.x;
          if (i < slab_units) {
            const unsigned wd = i << 2;
            const unsigned row = a.div_L.div(wd);
            unsigned l = wd - row * a.L;
            unsigned d_local = a.div_H.div(row);
            unsigned h = row - d_local * a.H;
            const unsigned vals[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              tile[tm16_index(a, d_local, h, l)] = vals[k];
              if (++l == a.L) {
                l = 0;
                if (++h == a.H) { h = 0; ++d_local; }
              }
            }
          }
        }
      }
      __syncthreads();
      // shared -> worker: one K vector and one V vector per (layer, h, g)
      for (unsigned o = threadIdx.x; o < n_out; o += blockDim.x) {
        const unsigned l = a.div_HG.div(o);
        const unsigned hg = o - l * HG;
        const unsigned h = a.div_Gs.div(hg);
        const unsigned g = hg - h * a.Gs;
        const unsigned* src = tile + hg * a.Lp + l;    // (h*Gs + g)*Lp + l, j = 0
        unsigned wv[8];
#pragma unroll
        for (unsigned j = 0; j < 8; ++j) wv[j] = src[j * j_pitch];
        uint4 kv, vv;
        kv.x = __byte_perm(wv[0], wv[1], 0x5410); vv.x = __byte_perm(wv[0], wv[1], 0x7632);
        kv.y = __byte_perm(wv[2], wv[3], 0x5410); vv.y = __byte_perm(wv[2], wv[3], 0x7632);
        kv.z = __byte_perm(wv[4], wv[5], 0x5410); vv.z = __byte_perm(wv[4], wv[5], 0x7632);
        kv.w = __byte_perm(wv[6], wv[7], 0x5410); vv.w = __byte_perm(wv[6], wv[7], 0x7632);
        unsigned short* kdst = work_tok + (2ull * l) * plane_elems + h * a.D + g * 8;
        st_stream16(kdst, kv);
        st_stream16(kdst + plane_elems, vv);
      }
      __syncthreads();
    } else {
      for (unsigned o = threadIdx.x; o < n_out; o += blockDim.x) {
        const unsigned l = a.div_HG.div(o);
        const unsigned hg = o - l * HG;
        const unsigned h = a.div_Gs.div(hg);
        const unsigned g = hg - h * a.Gs;
        const unsigned short* ksrc = work_tok + (2ull * l) * plane_elems + h * a.D + g * 8;
        const uint4 kv = ld_stream16(ksrc);
        const uint4 vv = ld_stream16(ksrc + plane_elems);
        const unsigned ks[4] = {kv.x, kv.y, kv.z, kv.w};
        const unsigned vs[4] = {vv.x, vv.y, vv.z, vv.w};
        unsigned* dst = tile + hg * a.Lp + l;
#pragma unroll
        for (unsigned q = 0; q < 4; ++q) {
          dst[(2 * q) * j_pitch] = __byte_perm(ks[q], vs[q], 0x5410);
          dst[(2 * q + 1) * j_pitch] = __byte_perm(ks[q], vs[q], 0x7632);
        }
      }
      __syncthreads();
      for (unsigned i = threadIdx.x; i < slab_units; i += blockDim.x) {
        const unsigned wd = i << 2;
        const unsigned row = a.div_L.div(wd);
        unsigned l = wd - row * a.L;
        unsigned d_local = a.div_H.div(row);
        unsigned h = row - d_local * a.H;
        unsigned vals[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          vals[k] = tile[tm16_index(a, d_local, h, l)];
          if (++l == a.L) {
            l = 0;
            if (++h == a.H) { h = 0; ++d_local; }
          }
        }
        st_stream16(pool_p + i, make_uint4(vals[0], vals[1], vals[2], vals[3]));
      }
      __syncthreads();
    }
  }
}


// ---------------------------------------------------------------------------
// Token-major pool, 2-byte elements, n_layers a multiple of 4: 16-byte shared
// memory accesses on both sides.
//
// The slab (Gs groups of 8 d, Hs consecutive heads, all layers of one token) is kept
// in its pool order, one row per (d, h) of L words, padded to RU 16-byte units (a
// multiple of 8).  The unit at position q of row (d, h) is stored at q ^ (hg & 7),
// hg = h*Gs + d/8 the index of the row's (head, d-group) within the slab.  Pool side:
// 16-byte units copied straight through, one contiguous run of Hs*L words per d (the
// whole slab is one run when Hs = H); cp.async on gather, so the next slab loads while
// this one is written out.
// Worker side: thread (lq, h, g) reads the 8 rows j = 0..7 of its (h, g) at unit
// lq -- the 8 lanes of a quarter warp have 8 consecutive hg, so the XOR sends them
// to 8 different bank groups -- and turns the 8 x 4 (K,V) words into 4 K vectors and
// 4 V vectors of 8 consecutive d, each part of a contiguous run of the warp.
// The scatter stages the worker vectors instead (MODE 2 below) and keeps the tile form
// (MODE 1) selectable for comparison.
// ---------------------------------------------------------------------------
struct TokenMajor16vArgs {
  const uint4* recs;
  const bikv_request_desc* reqs;
  PoolDev pool;
  unsigned n_items;      // n_pages * page_tokens * slabs
  unsigned page_tokens;
  unsigned slabs;        // (G / Gs) * hslabs
  unsigned hslabs;       // H / Hs
  unsigned Gs;           // d-groups (of 8) per slab
  unsigned Hs;           // heads per slab (divides H)
  unsigned H, D, L;
  unsigned LU;           // L / 4: 16-byte units per row
  unsigned RU;           // padded row pitch in units, a multiple of 8
  unsigned d_skip;       // (H - Hs) * LU: pool units between the runs of consecutive d
  int single;            // 1: one item per CTA, no ring (the grid is then as large as the work)
  FastDiv div_LU, div_Hs, div_HG, div_Gs, div_slabs, div_hslabs, div_ptok;
  unsigned long long token_bytes;  // D*H*L*4
  int to_pool;
  int* status;
  unsigned n_requests;
  unsigned long long total_pages;
};

struct TmItem {
  uint4* pool_p;
  unsigned short* work_tok;
  unsigned long long plane_elems;
  bool valid;
};

template <bool SPLIT>
__device__ __forceinline__ TmItem tm16v_item(const TokenMajor16vArgs& a, unsigned w) {
  TmItem it;
  it.valid = false;
  if (w >= a.n_items) return it;
  const unsigned t = a.div_slabs.div(w);
  const unsigned slab = w - t * a.slabs;
  const unsigned page = a.div_ptok.div(t);
  const unsigned tok = t - page * a.page_tokens;
  const uint4 r = __ldg(a.recs + page);
  if (!record_ok(r, a.n_requests, a.page_tokens, a.total_pages, a.status)) return it;
  if (tok >= r.y) return it;
  const unsigned id = r.x;
  unsigned shard;
  unsigned long long local;
  if (a.pool.rule == BIKV_SHARD_MOD) {
    shard = id % (unsigned)a.pool.n_shards;
    local = id / (unsigned)a.pool.n_shards;
  } else {
    shard = (unsigned)(id / a.pool.pages_per_shard);
    local = id % a.pool.pages_per_shard;
  }
  const unsigned gslab = SPLIT ? a.div_hslabs.div(slab) : slab;
  const unsigned h0 = SPLIT ? (slab - gslab * a.hslabs) * a.Hs : 0u;   // first head of the slab
  const unsigned d0 = gslab * a.Gs * 8;                                // first d of the slab
  it.pool_p = reinterpret_cast<uint4*>(a.pool.base[shard] + (local * a.page_tokens + tok) * a.token_bytes) +
              ((unsigned long long)d0 * a.H + h0) * a.LU;
  const longlong2 rq = __ldg(reinterpret_cast<const longlong2*>(a.reqs + r.z));
  if (!window_ok(r, (unsigned long long)rq.x, rq.y, a.status)) return it;
  const unsigned row_elems = a.H * a.D;
  it.work_tok = reinterpret_cast<unsigned short*>(rq.x) + (unsigned long long)(r.w + tok) * row_elems +
                h0 * a.D + d0;
  it.plane_elems = (unsigned long long)rq.y * row_elems;
  it.valid = true;
  return it;
}

// Unit i of the slab (row = i / LU = d_local*Hs + h, q = i % LU): its index in shared
// memory and its offset from the slab's first unit in the pool.
template <bool SPLIT>
__device__ __forceinline__ void tm16v_unit(const TokenMajor16vArgs& a, unsigned i, unsigned& smem_unit,
                                           unsigned& pool_unit) {
  const unsigned row = a.div_LU.div(i);
  const unsigned q = i - row * a.LU;
  const unsigned d_local = a.div_Hs.div(row);
  const unsigned h = row - d_local * a.Hs;
  const unsigned hg = h * a.Gs + (d_local >> 3);
  smem_unit = row * a.RU + (q ^ (hg & 7));
  pool_unit = SPLIT ? i + d_local * a.d_skip : i;
}

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// SPLIT = the slab holds fewer heads than the pool row (Hs < H).  MODE: 0 = gather,
// 1 = scatter through the transposed tile, 2 = scatter through staged worker rows.
// RING3: three buffers in the cp.async ring of modes 0 and 2 instead of two.
template <bool SPLIT, int MODE, bool RING3>
__global__ void __launch_bounds__(256) k_token_major16v(const __grid_constant__ TokenMajor16vArgs a) {
  extern __shared__ __align__(16) uint4 tm16v_tile[];
  const unsigned HG = a.Hs * a.Gs;
  const unsigned rows = a.Gs * 8 * a.Hs;
  const unsigned slab_units = rows * a.LU;
  const unsigned tile_units = rows * a.RU;
  const unsigned n_out = a.LU * HG;

  if constexpr (MODE == 0) {
    // Gather: two tiles; the slab of the next item streams in with cp.async while
    // the current one is transposed out.
    auto load = [&](const TmItem& it, uint4* tile) {
      if (!it.valid) return;
      const uint32_t base = smem_u32(tile);
      for (unsigned i = threadIdx.x; i < slab_units; i += blockDim.x) {
        unsigned su, pu;
        tm16v_unit<SPLIT>(a, i, su, pu);
        cp_async16(base + su * 16u, it.pool_p + pu);
      }
    };
    auto emit = [&](const TmItem& cur, const uint4* tile) {
      if (!cur.valid) return;
      for (unsigned o = threadIdx.x; o < n_out; o += blockDim.x) {
        const unsigned lq = a.div_HG.div(o);
        const unsigned hg = o - lq * HG;
        const unsigned h = a.div_Gs.div(hg);
        const unsigned g = hg - h * a.Gs;
        const unsigned q = lq ^ (hg & 7);
        uint4 wv[8];
#pragma unroll
        for (unsigned j = 0; j < 8; ++j) wv[j] = tile[(((g << 3) + j) * a.Hs + h) * a.RU + q];
        unsigned short* dst = cur.work_tok + (8ull * lq) * cur.plane_elems + h * a.D + g * 8;
#pragma unroll
        for (unsigned c = 0; c < 4; ++c) {
          const unsigned x0 = (&wv[0].x)[c], x1 = (&wv[1].x)[c], x2 = (&wv[2].x)[c], x3 = (&wv[3].x)[c];
          const unsigned x4 = (&wv[4].x)[c], x5 = (&wv[5].x)[c], x6 = (&wv[6].x)[c], x7 = (&wv[7].x)[c];
          uint4 kv, vv;
          kv.x = __byte_perm(x0, x1, 0x5410); vv.x = __byte_perm(x0, x1, 0x7632);
          kv.y = __byte_perm(x2, x3, 0x5410); vv.y = __byte_perm(x2, x3, 0x7632);
          kv.z = __byte_perm(x4, x5, 0x5410); vv.z = __byte_perm(x4, x5, 0x7632);
          kv.w = __byte_perm(x6, x7, 0x5410); vv.w = __byte_perm(x6, x7, 0x7632);
          st_stream16(dst + (2ull * c) * cur.plane_elems, kv);
          st_stream16(dst + (2ull * c + 1) * cur.plane_elems, vv);
        }
      }
    };
    if (a.single) {
      // One item per CTA: load, wait, write out, exit.  The CTAs that share an SM cover each
      // other's latencies and the block scheduler hands out the items.
      const TmItem it = tm16v_item<SPLIT>(a, blockIdx.x);
      if (!it.valid) return;
      load(it, tm16v_tile);
      cp_async_commit();
      cp_async_wait_all();
      __syncthreads();
      emit(it, tm16v_tile);
      return;
    }
    unsigned w = blockIdx.x;
    if constexpr (RING3) {
      // Three tiles: the slabs of the next two items are in flight while the current one
      // is transposed out.
      TmItem cur = tm16v_item<SPLIT>(a, w);
      TmItem nxt = tm16v_item<SPLIT>(a, w + gridDim.x);
      load(cur, tm16v_tile);
      cp_async_commit();
      load(nxt, tm16v_tile + tile_units);
      cp_async_commit();
      unsigned buf = 0;
      while (w < a.n_items) {
        const TmItem after = tm16v_item<SPLIT>(a, w + 2 * gridDim.x);
        const unsigned b2 = buf >= 1 ? buf - 1 : 2;   // (buf + 2) % 3
        load(after, tm16v_tile + b2 * tile_units);
        cp_async_commit();
        asm volatile("cp.async.wait_group 2;" ::: "memory");
        __syncthreads();
        emit(cur, tm16v_tile + buf * tile_units);
        __syncthreads();  // this tile is the target of the next iteration's load
        cur = nxt;
        nxt = after;
        w += gridDim.x;
        buf = buf == 2 ? 0 : buf + 1;
      }
      cp_async_wait_all();
      return;
    }
    TmItem cur = tm16v_item<SPLIT>(a, w);
    unsigned buf = 0;
    load(cur, tm16v_tile);
    cp_async_commit();
    while (w < a.n_items) {
      const unsigned w_next = w + gridDim.x;
      const TmItem nxt = tm16v_item<SPLIT>(a, w_next);
      load(nxt, tm16v_tile + (buf ^ 1) * tile_units);
      cp_async_commit();
      // everything but the group just committed has landed
      asm volatile("cp.async.wait_group 1;" ::: "memory");
      __syncthreads();
      emit(cur, tm16v_tile + buf * tile_units);
      __syncthreads();  // the tile may be overwritten by the load after next
      cur = nxt;
      w = w_next;
      buf ^= 1;
    }
    cp_async_wait_all();
    return;
  }

  if constexpr (MODE == 2) {
    // Scatter through staged worker rows: the 16-byte worker vectors of the slab stream
    // into shared memory with cp.async in worker order, [plane][head, d-group], the unit
    // of (plane, hg) at hg ^ (plane/8 & 7) so that the reads below spread over the banks;
    // the rows of the next item load while thread (4 layers, head, d-group) reads its 4 K
    // and 4 V vectors of the current one, turns them into the 8 pool units (8 d x 4
    // layers of K,V) and stores those straight to the pool: lanes run along the layers
    // of a row, then along the heads, so a warp's stores form contiguous runs.
    const unsigned HGp = (HG + 7u) & ~7u;
    const unsigned stage_units = 8 * a.LU * HGp;
    auto load = [&](const TmItem& it, uint4* stage) {
      if (!it.valid) return;
      const uint32_t base = smem_u32(stage);
      for (unsigned i = threadIdx.x; i < slab_units; i += blockDim.x) {
        const unsigned p = a.div_HG.div(i);          // plane 2*layer + kv
        const unsigned hg = i - p * HG;
        const unsigned h = a.div_Gs.div(hg);
        const unsigned g = hg - h * a.Gs;
        const unsigned su = p * HGp + (hg ^ ((p >> 3) & 7));
        cp_async16(base + su * 16u, it.work_tok + (unsigned long long)p * it.plane_elems + h * a.D + g * 8);
      }
    };
    auto emit = [&](const TmItem& cur, const uint4* stage) {
      if (!cur.valid) return;
      for (unsigned o = threadIdx.x; o < n_out; o += blockDim.x) {
        const unsigned t = a.div_LU.div(o);
        const unsigned lq = o - t * a.LU;
        const unsigned g = a.div_Hs.div(t);
        const unsigned h = t - g * a.Hs;
        const unsigned hg = h * a.Gs + g;
        const uint4* src = stage + (8 * lq) * HGp + (hg ^ (lq & 7));
        uint4 kv[4], vv[4];
#pragma unroll
        for (unsigned c = 0; c < 4; ++c) {
          kv[c] = src[(2 * c) * HGp];
          vv[c] = src[(2 * c + 1) * HGp];
        }
        const unsigned row_pitch = a.H * a.LU;   // pool units between d and d + 1
        uint4* dst = cur.pool_p + ((g << 3) * a.H + h) * a.LU + lq;
#pragma unroll
        for (unsigned j = 0; j < 8; ++j) {
          // word c of row j: K_j of layer 4*lq + c in the low half, V_j in the high half
          uint4 out;
          const unsigned sel = (j & 1) ? 0x7632 : 0x5410;
          out.x = __byte_perm((&kv[0].x)[j >> 1], (&vv[0].x)[j >> 1], sel);
          out.y = __byte_perm((&kv[1].x)[j >> 1], (&vv[1].x)[j >> 1], sel);
          out.z = __byte_perm((&kv[2].x)[j >> 1], (&vv[2].x)[j >> 1], sel);
          out.w = __byte_perm((&kv[3].x)[j >> 1], (&vv[3].x)[j >> 1], sel);
          st_stream16(dst + j * row_pitch, out);
        }
      }
    };
    if (a.single) {
      // One item per CTA: load, wait, write out, exit.  The CTAs that share an SM cover each
      // other's latencies and the block scheduler hands out the items.
      const TmItem it = tm16v_item<SPLIT>(a, blockIdx.x);
      if (!it.valid) return;
      load(it, tm16v_tile);
      cp_async_commit();
      cp_async_wait_all();
      __syncthreads();
      emit(it, tm16v_tile);
      return;
    }
    unsigned w = blockIdx.x;
    if constexpr (RING3) {   // the worker vectors of the next two items in flight
      TmItem cur = tm16v_item<SPLIT>(a, w);
      TmItem nxt = tm16v_item<SPLIT>(a, w + gridDim.x);
      load(cur, tm16v_tile);
      cp_async_commit();
      load(nxt, tm16v_tile + stage_units);
      cp_async_commit();
      unsigned buf = 0;
      while (w < a.n_items) {
        const TmItem after = tm16v_item<SPLIT>(a, w + 2 * gridDim.x);
        const unsigned b2 = buf >= 1 ? buf - 1 : 2;   // (buf + 2) % 3
        load(after, tm16v_tile + b2 * stage_units);
        cp_async_commit();
        asm volatile("cp.async.wait_group 2;" ::: "memory");
        __syncthreads();
        emit(cur, tm16v_tile + buf * stage_units);
        __syncthreads();  // this stage is the target of the next iteration's load
        cur = nxt;
        nxt = after;
        w += gridDim.x;
        buf = buf == 2 ? 0 : buf + 1;
      }
      cp_async_wait_all();
      return;
    }
    TmItem cur = tm16v_item<SPLIT>(a, w);
    unsigned buf = 0;
    load(cur, tm16v_tile);
    cp_async_commit();
    while (w < a.n_items) {
      const unsigned w_next = w + gridDim.x;
      const TmItem nxt = tm16v_item<SPLIT>(a, w_next);
      load(nxt, tm16v_tile + (buf ^ 1) * stage_units);
      cp_async_commit();
      asm volatile("cp.async.wait_group 1;" ::: "memory");
      __syncthreads();
      emit(cur, tm16v_tile + buf * stage_units);
      __syncthreads();  // the stage may be overwritten by the load after next
      cur = nxt;
      w = w_next;
      buf ^= 1;
    }
    cp_async_wait_all();
    return;
  }

  // Scatter: worker -> shared (transposing) -> pool (straight through).  One tile: CTAs
  // sharing the SM cover each other's phases (a two-tile version that read the next item's
  // rows while the current tile drained halved the resident CTAs and measured slower,
  // 0.64 against 0.79 of the HBM copy peak at 80 layers x 8 heads).
  for (unsigned w = blockIdx.x; w < a.n_items; w += gridDim.x) {
    const TmItem it = tm16v_item<SPLIT>(a, w);
    if (!it.valid) continue;  // uniform across the CTA
    uint4* tile = tm16v_tile;
    for (unsigned o = threadIdx.x; o < n_out; o += blockDim.x) {
      const unsigned lq = a.div_HG.div(o);
      const unsigned hg = o - lq * HG;
      const unsigned h = a.div_Gs.div(hg);
      const unsigned g = hg - h * a.Gs;
      const unsigned q = lq ^ (hg & 7);
      const unsigned short* src = it.work_tok + (8ull * lq) * it.plane_elems + h * a.D + g * 8;
      uint4 kv[4], vv[4];
#pragma unroll
      for (unsigned c = 0; c < 4; ++c) {
        kv[c] = ld_stream16(src + (2ull * c) * it.plane_elems);
        vv[c] = ld_stream16(src + (2ull * c + 1) * it.plane_elems);
      }
#pragma unroll
      for (unsigned j = 0; j < 8; ++j) {
        // word c of row j: K_j of layer 4*lq + c in the low half, V_j in the high half
        uint4 out;
        const unsigned sel = (j & 1) ? 0x7632 : 0x5410;
        out.x = __byte_perm((&kv[0].x)[j >> 1], (&vv[0].x)[j >> 1], sel);
        out.y = __byte_perm((&kv[1].x)[j >> 1], (&vv[1].x)[j >> 1], sel);
        out.z = __byte_perm((&kv[2].x)[j >> 1], (&vv[2].x)[j >> 1], sel);
        out.w = __byte_perm((&kv[3].x)[j >> 1], (&vv[3].x)[j >> 1], sel);
        tile[(((g << 3) + j) * a.Hs + h) * a.RU + q] = out;
      }
    }
    __syncthreads();
    for (unsigned i = threadIdx.x; i < slab_units; i += blockDim.x) {
      unsigned su, pu;
      tm16v_unit<SPLIT>(a, i, su, pu);
      st_stream16(it.pool_p + pu, tile[su]);
    }
    __syncthreads();
  }
}

}  // namespace bikv
