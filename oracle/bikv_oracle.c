/*
 * Plain-C restatement of the KV-page path.  TEST INFRASTRUCTURE ONLY: an independent
 * second statement of what oracle/bikv_oracle.py states with torch slicing, so that the
 * two can be checked against each other.  Byte loops, no vector code, no threads.
 *
 *  - plan:   DistributedStorage/kvcache.py:158-174 (running token offset per destination,
 *            short last page of an item)
 *  - copy:   SharedMemory/CUDA_Shared/copy_kernel.cu:10-36 applied per valid token, with the
 *            pool layouts of include/bikv.h and the worker layout [layer][kv][token][head][dim]
 *  - flat:   copy_kernel.cu:10-36 as is (element offsets, whole pages)
 */
#include <stdint.h>
#include <string.h>

typedef struct { int32_t page_id, valid_tokens, request, token_offset; } rec_t;

int64_t c_plan_records(const int32_t* pages_flat, const int64_t* begin, const int32_t* item_tokens,
                       const int32_t* item_request, int32_t n_items, int32_t page_tokens,
                       int64_t* request_tokens, rec_t* out) {
  int64_t n = 0;
  for (int32_t it = 0; it < n_items; ++it) {
    int32_t req = item_request ? item_request[it] : 0;
    int64_t count = begin[it + 1] - begin[it];
    for (int64_t k = 0; k < count; ++k) {
      int32_t size = page_tokens;
      if (k == count - 1 && item_tokens[it] % page_tokens != 0) size = item_tokens[it] % page_tokens;
      out[n].page_id = pages_flat[begin[it] + k];
      out[n].valid_tokens = size;
      out[n].request = req;
      out[n].token_offset = (int32_t)request_tokens[req];
      request_tokens[req] += size;
      ++n;
    }
  }
  return n;
}

/* Byte offset of element (l, kv, t, h, d) of pool page `local` in the given layout. */
static int64_t pool_offset(int layout, int64_t local, int L, int H, int D, int P, int elt,
                           int l, int kv, int t, int h, int d) {
  if (layout == 0) /* paged: [page][L][2][P][H][D] */
    return ((((((int64_t)local * L + l) * 2 + kv) * P + t) * H + h) * D + d) * elt;
  /* token-major: [token][D][H][L][2] */
  return (((((local * (int64_t)P + t) * D + d) * H + h) * L + l) * 2 + kv) * (int64_t)elt;
}

/* direction 0: pool -> worker (gather); 1: worker -> pool (scatter). */
void c_move(unsigned char* const* shards, int n_shards, int64_t pages_per_shard, int rule, int layout,
            int L, int H, int D, int P, int elt, const rec_t* recs, int64_t n_recs,
            unsigned char* const* workers, const int64_t* worker_tokens, int direction) {
  for (int64_t i = 0; i < n_recs; ++i) {
    int64_t id = recs[i].page_id;
    int64_t shard = rule == 0 ? id % n_shards : id / pages_per_shard;
    int64_t local = rule == 0 ? id / n_shards : id % pages_per_shard;
    unsigned char* pool = shards[shard];
    unsigned char* work = workers[recs[i].request];
    int64_t T = worker_tokens[recs[i].request];
    for (int l = 0; l < L; ++l)
      for (int kv = 0; kv < 2; ++kv)
        for (int t = 0; t < recs[i].valid_tokens; ++t)
          for (int h = 0; h < H; ++h)
            for (int d = 0; d < D; ++d) {
              int64_t po = pool_offset(layout, local, L, H, D, P, elt, l, kv, t, h, d);
              int64_t wo = (((((int64_t)l * 2 + kv) * T + recs[i].token_offset + t) * H + h) * D + d) * elt;
              if (direction == 0) memcpy(work + wo, pool + po, (size_t)elt);
              else memcpy(pool + po, work + wo, (size_t)elt);
            }
  }
}

void c_copy_pages_flat(const unsigned char* src, unsigned char* dst, const int64_t* src_off,
                       const int64_t* dst_off, int64_t n_pages, int64_t page_elems, int elt) {
  for (int64_t i = 0; i < n_pages; ++i)
    for (int64_t e = 0; e < page_elems; ++e)
      memcpy(dst + (dst_off[i] + e) * elt, src + (src_off[i] + e) * elt, (size_t)elt);
}
