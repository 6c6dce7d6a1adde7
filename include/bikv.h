/*
 * bikv.h -- C ABI of the B200 KV-page data path (libbikv.so).
 *
 * The library moves KV-cache pages between sharded page pools (the KVCache
 * shards of Bi-KV) and a worker's contiguous per-request KV tensors:
 *
 *   gather   pool pages  -> worker KV   (task type SEND in the reference)
 *   scatter  worker KV   -> pool pages  (task type RECV in the reference)
 *
 * Everything crosses this boundary as plain pointers and sizes; no torch or
 * C++ types appear.  All device work is asynchronous on the stream the caller
 * passes (a cudaStream_t cast to void*; NULL is the legacy default stream).
 * Unless a function says otherwise the library allocates no device memory and
 * never frees caller memory.
 *
 * Each entry point names the reference interface it replaces, as
 * path:line inside the Bi-KV project.
 */
#ifndef BIKV_H_
#define BIKV_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BIKV_ABI_VERSION 1
#define BIKV_MAX_SHARDS 16

/* ---- status codes (0 = success, negative = error) ----------------------- */
enum bikv_status {
  BIKV_OK = 0,
  BIKV_ERR_BAD_ARG = -1,        /* null pointer, non-positive size, unknown enum        */
  BIKV_ERR_PAGE_RANGE = -2,     /* page id outside the pool                              */
  BIKV_ERR_DST_RANGE = -3,      /* token window outside the request's KV tensor          */
  BIKV_ERR_ALIGNMENT = -4,      /* a base or a row is not 16-byte aligned                */
  BIKV_ERR_PEER = -5,           /* peer access / IPC mapping could not be set up         */
  BIKV_ERR_CUDA = -6,           /* a CUDA call failed; see bikv_last_cuda_error()        */
  BIKV_ERR_OVERLAP = -7,        /* two records of a scatter plan write the same page     */
  BIKV_ERR_DEVICE_TIMEOUT = -8, /* a bounded wait inside a kernel ran out                */
  BIKV_ERR_TOO_LARGE = -9,      /* plan or size beyond a documented maximum              */
  BIKV_ERR_PLAN = -10           /* plan inconsistent (page count vs token count, ...)    */
};

/* ---- pool page layouts --------------------------------------------------- */
enum bikv_pool_layout {
  /* page = [layer][kv][page_token][head][dim]; every (page, layer, kv) plane
   * is one contiguous run of page_tokens*heads*dim elements.               */
  BIKV_POOL_PAGED = 0,
  /* The reference pool: page = page_tokens consecutive tokens, each token
   * laid out [dim][head][layer][kv] (DistributedStorage/kvcache.py:38-43 with
   * token_shape of Model/qwen2.py:519-522).                                 */
  BIKV_POOL_TOKEN_MAJOR = 1
};

/* How a global page id maps to (shard, page inside the shard). */
enum bikv_shard_rule {
  BIKV_SHARD_MOD = 0,   /* shard = id % n_shards, local = id / n_shards                */
  BIKV_SHARD_BLOCK = 1  /* shard = id / pages_per_shard, local = id % pages_per_shard
                           (the reference's item-granular placement: id =
                           cache_worker * pages_per_shard + page)                      */
};

/* Copy engine selection for the paged layout. */
enum bikv_variant {
  BIKV_VARIANT_AUTO = 0, /* ld/st for a single-shard pool, bulk ring for a sharded one
                            (override with the "auto_variant" knob: 1 or 2; 0 = this rule) */
  BIKV_VARIANT_LDST = 1, /* warp per chunk, 16-byte ld/st                              */
  BIKV_VARIANT_BULK = 2  /* cp.async.bulk global->shared->global ring per CTA          */
};

typedef struct bikv_geometry {
  int32_t n_layers;
  int32_t n_kv_heads;
  int32_t head_dim;
  int32_t page_tokens;
  int32_t elt_bytes;   /* 2 for fp16 / bf16 (bit passthrough), 1 and 4 also accepted */
  int32_t pool_layout; /* enum bikv_pool_layout */
} bikv_geometry;

/* One page of a plan.  `request` selects the worker KV tensor, `token_offset`
 * the first token inside it, `valid_tokens` (1..page_tokens) how many tokens of
 * the page carry data (a request's last page may be partial). */
typedef struct bikv_page_rec {
  int32_t page_id;
  int32_t valid_tokens;
  int32_t request;
  int32_t token_offset;
} bikv_page_rec;

/* A worker-side KV tensor, layout [layer][kv][tokens][head][dim]. */
typedef struct bikv_request_desc {
  void* base;
  int64_t tokens;
} bikv_request_desc;

/* The sharded pool as one worker GPU sees it: shard_base[s] is a device pointer
 * valid on the calling GPU (its own memory, or a peer mapping). */
typedef struct bikv_pool_desc {
  void* shard_base[BIKV_MAX_SHARDS];
  int32_t n_shards;
  int32_t shard_rule; /* enum bikv_shard_rule */
  int64_t pages_per_shard;
} bikv_pool_desc;

/* ---- library ------------------------------------------------------------- */
int bikv_version(void);
const char* bikv_strerror(int status);
/* cudaError_t of the last failing CUDA call on this thread (0 if none). */
int bikv_last_cuda_error(void);
/* Number of kernels this library has launched in this process. */
int64_t bikv_launch_count(void);
/* Tuning knobs: "ldst_ctas_per_sm", "bulk_ctas_per_sm", "bulk_stages", "bulk_span", "ldst_wide",
 * "ldst_seg_bytes", "tm_single",
 * "seg_bytes", "auto_variant", "ldst_threads", "tm_threads", "tm16_threads", "tm_max_groups",
 * "tm_tile_kib", "tm_split_tile_kib", "tm_max_heads", "tm_scatter_staged", "tm_gather_stages",
 * "tm_scatter_stages".
 * Returns BIKV_ERR_BAD_ARG for unknown names or values out of range. */
int bikv_set_tuning(const char* name, int64_t value);
int64_t bikv_get_tuning(const char* name);

/* ---- plan (host) --------------------------------------------------------- */
/*
 * Builds page records from a coordinator plan.  Replaces the index loops of
 * KVCache.shared_data_batch_pages (DistributedStorage/kvcache.py:158-196):
 * items are walked in order, each page of an item gets the running token
 * offset of its request, and the last page of an item whose token count is
 * not a multiple of page_tokens carries only the remainder.
 *   pages_flat      all items' page ids, concatenated
 *   item_page_begin n_items+1 offsets into pages_flat
 *   item_tokens     token count per item
 *   item_request    destination tensor per item, or NULL (all request 0)
 *   item_shard      cache_worker per item for BIKV_SHARD_BLOCK (page id becomes
 *                   shard*pages_per_shard + page), or NULL
 *   request_tokens  in/out: running token count per request (start at 0)
 * Returns the number of records written (>= 0) or a negative status.
 */
int64_t bikv_plan_build(const int32_t* pages_flat, const int64_t* item_page_begin,
                        const int32_t* item_tokens, const int32_t* item_request,
                        const int32_t* item_shard, int64_t pages_per_shard,
                        int32_t n_items, int32_t page_tokens,
                        int64_t* request_tokens, int32_t n_requests,
                        bikv_page_rec* out, int64_t out_capacity);

/*
 * Checks a host-resident plan before anything is launched: page ids inside the
 * pool, valid_tokens in 1..page_tokens, token windows inside their request,
 * geometry sane, and (check_overlap != 0) no pool page named twice -- required
 * for scatter.  The reference performs no such check (copy_kernel.cu:68-129
 * launches unconditionally).  request_base may be NULL (alignment unchecked).
 */
int bikv_plan_validate(const bikv_page_rec* recs, int64_t n_pages,
                       const bikv_request_desc* requests, int32_t n_requests,
                       const bikv_pool_desc* pool, const bikv_geometry* geom,
                       int check_overlap);

/*
 * The shard-driven SEND: in the reference the KVCache shard is the active side of a
 * gather and writes into the worker's buffer (KVCache.send_data_batch -> post_rdma_write,
 * DistributedStorage/kvcache.py:96-113).  Here the GPU that owns a page may do the same
 * with bikv_gather, given a plan that holds only ITS pages and a request table whose
 * bases are the workers' tensors as mapped on that GPU.  This builds that plan: from
 * every worker's records it keeps those whose page lives on shard `owner` and renumbers
 * `request` into one table over all workers (worker w's request i becomes
 * requests_per_worker[0] + ... + requests_per_worker[w-1] + i).  Rows of different
 * workers are interleaved in proportion to their counts (a worker's own order is kept):
 * a kernel sweeps its plan front to back with all CTAs side by side, so rows grouped by
 * destination would send every owner's traffic to one worker at a time.
 *   tables[w], n_rows[w]   worker w's records (host memory)
 * Returns the number of records written, or a negative status (BIKV_ERR_TOO_LARGE when
 * `out_capacity` is too small; the sum of n_rows always suffices).
 */
int64_t bikv_plan_split_by_owner(const bikv_page_rec* const* tables, const int64_t* n_rows,
                                 const int32_t* requests_per_worker, int32_t n_workers, int32_t owner,
                                 int32_t n_shards, int64_t pages_per_shard, int32_t shard_rule,
                                 bikv_page_rec* out, int64_t out_capacity);

/*
 * The rule every kernel applies to a worker-side base address -- a request's KV
 * tensor (bikv_request_desc.base) or a layer tensor of a paged worker cache --
 * before it forms an address from it: BIKV_ERR_BAD_ARG for NULL,
 * BIKV_ERR_ALIGNMENT unless 16-byte aligned, else BIKV_OK.  Host code and device
 * code share the one function, so a caller that keeps its tables in device memory
 * can pre-check them with exactly the kernels' rule.  The reference checks nothing
 * of the kind (SharedMemory/CUDA_Shared/copy_kernel.cu:68-129 launches unchecked).
 */
int bikv_check_worker_base(const void* base);

/* ---- gather / scatter (device) ------------------------------------------- */
/*
 * Gather: for every record, pool page -> request KV window, converting the pool
 * layout into [layer][kv][tokens][head][dim].  Replaces
 * cuda_producer_copy_pages + block_per_page_copy_kernel
 * (SharedMemory/CUDA_Shared/copy_kernel.cu:10-36,68-129) and, when a shard base
 * is a peer mapping, the one-sided read of NetworkTransport/onesided_rdma.h:706-759.
 *   recs_dev / requests_dev  device arrays (n_pages / n_requests entries)
 *   status_dev               device int32[4], zeroed by the caller; word 0
 *                            receives a bikv_status if a bounded device wait
 *                            runs out, or if a record points outside the pool or
 *                            outside its worker tensor, or selects a request whose
 *                            base is NULL or not 16-byte aligned: the kernels check
 *                            every record and SKIP a bad one instead of touching memory
 *                            (records in device memory cannot be checked on the
 *                            host).  May be NULL for BIKV_VARIANT_LDST; bad records
 *                            are then skipped silently.
 */
int bikv_gather(const bikv_pool_desc* pool, const bikv_geometry* geom,
                const bikv_page_rec* recs_dev, int64_t n_pages,
                const bikv_request_desc* requests_dev, int32_t n_requests,
                int variant, int32_t* status_dev, void* stream);

/*
 * Scatter: the exact inverse index map of bikv_gather (request KV window ->
 * pool page; only valid_tokens tokens of a partial page are written).  The
 * reference has no kernel for this direction; it is implied by
 * KVCache.receive_data_batch (DistributedStorage/kvcache.py:116-130) and
 * Worker.send_kvcache_data_batch (Worker/Worker.py:193-218), and by the
 * one-sided write of NetworkTransport/onesided_rdma.h:652-704.
 */
int bikv_scatter(const bikv_pool_desc* pool, const bikv_geometry* geom,
                 const bikv_page_rec* recs_dev, int64_t n_pages,
                 const bikv_request_desc* requests_dev, int32_t n_requests,
                 int variant, int32_t* status_dev, void* stream);

/*
 * Host-plan forms: the plan lives in host memory (pinned for a truly
 * asynchronous upload).  The call validates it (validate != 0), copies it into
 * `plan_scratch_dev` (caller-owned device memory of at least
 * bikv_plan_scratch_bytes(n_pages, n_requests) bytes) on `stream`, and launches
 * the kernel behind it.  This is what KVCache.send_data_batch /
 * receive_data_batch (DistributedStorage/kvcache.py:96-130) call.
 * The host arrays must stay unchanged until the stream has passed the upload.
 */
int64_t bikv_plan_scratch_bytes(int64_t n_pages, int32_t n_requests);
int bikv_gather_h(const bikv_pool_desc* pool, const bikv_geometry* geom,
                  const bikv_page_rec* recs_host, int64_t n_pages,
                  const bikv_request_desc* requests_host, int32_t n_requests,
                  void* plan_scratch_dev, int64_t plan_scratch_bytes, int validate,
                  int variant, int32_t* status_dev, void* stream);
int bikv_scatter_h(const bikv_pool_desc* pool, const bikv_geometry* geom,
                   const bikv_page_rec* recs_host, int64_t n_pages,
                   const bikv_request_desc* requests_host, int32_t n_requests,
                   void* plan_scratch_dev, int64_t plan_scratch_bytes, int validate,
                   int variant, int32_t* status_dev, void* stream);

/*
 * Gather / scatter against a worker's PAGED KV instead of contiguous per-request
 * tensors: one tensor per layer, laid out [slot][kv][head][dim] with slot =
 * block * block_tokens + token -- the Worker's local_kvcache (Worker/Worker.py:68-78)
 * that the model's paged prefill reads (Model/qwen2.py:169-181,273-276).  Nothing in
 * the reference fills that cache from the pool; these entry points do it without an
 * intermediate tensor.  For record i, token t < valid_tokens of pool page page_id maps
 * to slot token_offset + t of every layer (rec.request is ignored).
 *   layer_bases_dev  device array of n_layers pointers (one tensor per layer)
 *   slots_per_layer  slots in each layer tensor (bounds for bikv_plan_validate_nhd)
 * BIKV_POOL_PAGED pools only (BIKV_ERR_BAD_ARG otherwise).
 */
int bikv_gather_nhd(const bikv_pool_desc* pool, const bikv_geometry* geom,
                    const bikv_page_rec* recs_dev, int64_t n_pages,
                    void* const* layer_bases_dev, int64_t slots_per_layer,
                    int32_t* status_dev, void* stream);
int bikv_scatter_nhd(const bikv_pool_desc* pool, const bikv_geometry* geom,
                     const bikv_page_rec* recs_dev, int64_t n_pages,
                     void* const* layer_bases_dev, int64_t slots_per_layer,
                     int32_t* status_dev, void* stream);
/* Host-side check of a paged-worker plan: page ids in the pool, valid_tokens in
 * 1..page_tokens, slots inside [0, slots_per_layer), and (check_overlap) no pool
 * page named twice. */
int bikv_plan_validate_nhd(const bikv_page_rec* recs, int64_t n_pages, int64_t slots_per_layer,
                           const bikv_pool_desc* pool, const bikv_geometry* geom, int check_overlap);

/*
 * Gather for callers that must not allocate.  No counterpart in the reference.
 *
 * Same meaning as bikv_gather_h, but the caller brings no plan staging buffer:
 * the plan is uploaded into a fixed array that is part of this library's device
 * image (BIKV_STATIC_PLAN_BYTES, resident on every GPU that loads the library
 * until the process exits).  The call makes no cudaMalloc/cudaFree and calls no
 * allocating library routine, so it is usable from a process whose serving
 * engine has already reserved all of HBM for its KV pool (a later cudaMalloc
 * there fails or has to wait for memory to be given back), and from a handler on
 * the transfer path, where the device-wide synchronisation hidden inside
 * cudaMalloc/cudaFree would stall every other stream's copies.
 *
 * Limits: n_pages <= BIKV_STATIC_MAX_PAGES and n_requests <=
 * BIKV_STATIC_MAX_REQUESTS; larger plans are refused with BIKV_ERR_TOO_LARGE
 * before anything is copied or launched (split the plan, or use bikv_gather_h).
 * The first call on a device looks up the array's device address (with that
 * device current); make that first call outside any stream capture.  It is also
 * the moment the CUDA runtime may place the library's device image -- this array
 * included -- on the GPU (module loading is lazy by default), and that placement
 * needs free device memory: make one call per device at start-up, BEFORE the
 * engine reserves HBM, or it can fail with BIKV_ERR_CUDA (out of memory).  A call
 * with n_pages == 0 does exactly this set-up and launches nothing.
 * Every call on a device shares the one array: it still holds the previous
 * call's plan, nothing in it needs to start at zero (each call overwrites the
 * part it uses), and two calls whose GPU work overlaps -- different streams, or
 * different threads -- race on it.  Serialise them on one stream.
 * The caller still passes every input and output: pool, worker tensors,
 * status_dev (may be NULL for BIKV_VARIANT_LDST, as for bikv_gather_h).
 */
#define BIKV_STATIC_MAX_PAGES 32768
#define BIKV_STATIC_MAX_REQUESTS 1024
#define BIKV_STATIC_PLAN_BYTES (BIKV_STATIC_MAX_PAGES * 16 + BIKV_STATIC_MAX_REQUESTS * 16)
int bikv_gather_h_static(const bikv_pool_desc* pool, const bikv_geometry* geom,
                         const bikv_page_rec* recs_host, int64_t n_pages,
                         const bikv_request_desc* requests_host, int32_t n_requests,
                         int validate, int variant, int32_t* status_dev, void* stream);

/*
 * Flat page copy with the reference kernel's exact semantics
 * (SharedMemory/CUDA_Shared/copy_kernel.cu:10-36): for every page i and element
 * e < page_elems, dst[dst_off[i] + e] = src[src_off[i] + e]; offsets are in
 * ELEMENTS of elt_bytes.  `src` may be device memory (producer_copy_pages,
 * ipc_service.cpp:205-221) or pinned, device-mapped host memory
 * (zero_copy_page_kernel, copy_kernel.cu:39-66).  Offsets are device arrays.
 */
int bikv_copy_pages_flat(const void* src, void* dst, const int64_t* src_off_dev,
                         const int64_t* dst_off_dev, int64_t n_pages,
                         int64_t page_elems, int32_t elt_bytes, void* stream);

/*
 * One contiguous byte range, device to device (either side may be a peer
 * mapping).  Mirrors RDMAOneSidedEndpoint.post_rdma_write / post_rdma_read
 * (NetworkTransport/onesided_rdma.h:652-759) without the completion poll: the
 * copy is ordered on `stream`.
 */
int bikv_copy_range(void* dst, const void* src, int64_t bytes, void* stream);
/*
 * The same contiguous range moved by the GPU's copy engines instead of a kernel
 * (one cudaMemcpyAsync with unified addressing; either side may be device memory
 * of this GPU, a peer or IPC mapping, or pinned host memory).  It occupies no SM,
 * which suits the large single ranges of post_rdma_write / post_rdma_read
 * (NetworkTransport/onesided_rdma.h:652-759: one work request per contiguous
 * range), and it is the independent yardstick the benchmark holds the copy
 * kernels' NVLink throughput against.  Ordered on `stream`; launches no kernel.
 */
int bikv_copy_range_engine(void* dst, const void* src, int64_t bytes, void* stream);

/*
 * Diagnostic with no counterpart in the reference: launches one thread that waits
 * on a barrier nothing will complete, with a limit of limit_ns (at most 1 s), so
 * that the wait runs out and status_dev[0] receives BIKV_ERR_DEVICE_TIMEOUT -- the
 * path a copy ring takes when a bulk copy never arrives.  The kernel returns by
 * itself; the context stays usable.
 */
int bikv_selftest_wait_timeout(int32_t* status_dev, int64_t limit_ns, void* stream);

/*
 * Makes a host range (e.g. a mapping of a POSIX shared-memory block that two
 * processes share) page-locked and addressable by the GPUs, so that the copy
 * kernels and bikv_copy_range / bikv_copy_range_engine can read and write it in
 * place.  This is what stands in for ibv_reg_mr on the 'cpu' buffers of
 * RDMAOneSidedEndpoint (NetworkTransport/onesided_rdma.h:652-759 copy between
 * registered buffers; the registration itself is in its allocate_*_memory helpers).
 * Unregister before unmapping the range.
 */
int bikv_host_register(void* ptr, int64_t bytes);
int bikv_host_unregister(void* ptr);

/* ---- peer mapping -------------------------------------------------------- */
/* cudaDeviceCanAccessPeer / cudaDeviceEnablePeerAccess for in-process pools;
 * already-enabled is success. */
int bikv_can_access_peer(int device, int peer, int* can);
int bikv_enable_peer(int device, int peer);
/*
 * Cross-process exposure of a shard pool, the role of consumer_init /
 * producer_init (SharedMemory/CUDA_Shared/ipc_service.cpp:20-110) without the
 * POSIX shm block or the staging ring: export yields the 64-byte CUDA IPC
 * handle of the allocation that contains `ptr` plus ptr's offset inside it;
 * import maps it in another process and returns the mapped address of `ptr`.
 * bikv_pool_close takes the pointer import returned and the same offset.
 */
int bikv_pool_export(void* ptr, unsigned char handle[64], int64_t* offset);
int bikv_pool_import(const unsigned char handle[64], int64_t offset, void** ptr);
int bikv_pool_close(void* ptr, int64_t offset);

#ifdef __cplusplus
}
#endif
#endif /* BIKV_H_ */
