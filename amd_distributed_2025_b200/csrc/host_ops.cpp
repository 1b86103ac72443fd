#include "host_ops.h"

#include <ATen/Parallel.h>

#include <algorithm>
#include <atomic>
#include <cstring>
#include <vector>

namespace b200 {

namespace {

StatusWord ok_status() {
  StatusWord w;
  std::memset(&w, 0, sizeof(w));
  return w;
}

StatusWord bad_index(uint32_t phase, int detail, uint64_t epoch, uint64_t seen) {
  StatusWord w = ok_status();
  w.code = STATUS_BAD_INDEX;
  w.phase = phase;
  w.peer = -1;
  w.detail = detail;
  w.epoch = epoch;
  w.seen = seen;
  return w;
}

// Signal every rank, nearest higher rank first so that ranks do not all start on rank 0.
void signal_all(HostShmHeap& heap, int row, uint64_t epoch) {
  const int ws = heap.world_size();
  for (int i = 1; i <= ws; ++i) heap.signal(row, (heap.rank() + i) % ws, epoch);
}

StatusWord wait_all(HostShmHeap& heap, int row, uint64_t epoch, uint64_t timeout_ns, uint32_t phase) {
  for (int src = 0; src < heap.world_size(); ++src) {
    StatusWord w = heap.wait(row, src, epoch, timeout_ns, phase);
    if (w.code != STATUS_OK) return w;
  }
  return ok_status();
}

inline int64_t grain_for(int64_t row_bytes) {
  // about 256 KiB of payload per task: waking a pool thread costs more than copying less
  int64_t g = (256 << 10) / (row_bytes > 0 ? row_bytes : 1);
  return g < 1 ? 1 : g;
}

}  // namespace

StatusWord host_moe_dispatch(HostShmHeap& heap, const HostMoeLayout& lay, const HostMoeShape& s, const void* x,
                             const int32_t* indices, int num_tokens, int32_t* route, int32_t* expert_num_tokens,
                             uint64_t epoch, uint64_t timeout_ns) {
  const int ws = heap.world_size(), rank = heap.rank();
  const int E = s.num_experts, El = E / ws, n = num_tokens * s.topk;
  const int64_t row_bytes = (int64_t)s.hidden * host_dtype_bytes(s.in_dtype);
  StatusWord first = ok_status();

  // 1. count this rank's entries per expert and publish the row to every rank
  std::vector<int32_t> mine(E, 0);
  for (int i = 0; i < n; ++i) {
    const int e = indices[i];
    if (e < 0 || e >= E) {
      if (first.code == STATUS_OK) first = bad_index(PHASE_MOE_COUNTS, i, epoch, (uint64_t)(int64_t)e);
      continue;
    }
    ++mine[e];
  }
  for (int i = 1; i <= ws; ++i) {
    const int d = (rank + i) % ws;
    std::memcpy(heap.base(d) + lay.counts + (uint64_t)rank * E * sizeof(int32_t), mine.data(), E * sizeof(int32_t));
    heap.signal(FLAG_MOE_COUNTS, d, epoch);
  }
  StatusWord w = wait_all(heap, FLAG_MOE_COUNTS, epoch, timeout_ns, PHASE_MOE_COUNTS);
  if (w.code != STATUS_OK) return w;

  // 2. first slot of this rank inside every expert = rows of the lower ranks
  const int32_t* counts = reinterpret_cast<const int32_t*>(heap.base(rank) + lay.counts);
  std::vector<int32_t> next(E);
  for (int e = 0; e < E; ++e) {
    int32_t b = 0;
    for (int src = 0; src < rank; ++src) b += counts[src * E + e];
    next[e] = b;
  }
  for (int el = 0; el < El; ++el) {
    int32_t t = 0;
    for (int src = 0; src < ws; ++src) t += counts[src * E + rank * El + el];
    expert_num_tokens[el] = t;
  }

  // 3. slots in (token, k) order
  for (int i = 0; i < n; ++i) {
    const int e = indices[i];
    int32_t* r = route + 3 * (int64_t)i;
    r[0] = -1, r[1] = 0, r[2] = 0;
    if (e < 0 || e >= E) continue;
    const int slot = next[e]++;
    if (slot >= s.max_recv) {
      if (first.code == STATUS_OK) first = bad_index(PHASE_MOE_DATA, e, epoch, (uint64_t)slot);
      continue;
    }
    r[0] = e / El, r[1] = e % El, r[2] = slot;
  }

  // 4. rows and metadata straight into the owners' buffers
  const uint8_t* xb = static_cast<const uint8_t*>(x);
  at::parallel_for(0, n, grain_for(row_bytes), [&](int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) {
      const int32_t* r = route + 3 * i;
      if (r[0] < 0) continue;
      const int64_t cell = (int64_t)r[1] * s.max_recv + r[2];
      uint8_t* dst = heap.base(r[0]);
      std::memcpy(dst + lay.expert_x + cell * row_bytes, xb + (i / s.topk) * row_bytes, row_bytes);
      int32_t* meta = reinterpret_cast<int32_t*>(dst + lay.expert_meta) + cell * 5;
      meta[0] = indices[i];
      meta[1] = rank;
      meta[2] = (int32_t)(i / s.topk);
      meta[3] = (int32_t)(i % s.topk);
      meta[4] = 0;
    }
  });

  // 5. "my rows are in place" to everyone; leave when everyone's rows are here
  signal_all(heap, FLAG_MOE_DATA, epoch);
  w = wait_all(heap, FLAG_MOE_DATA, epoch, timeout_ns, PHASE_MOE_DATA);
  if (w.code != STATUS_OK) return w;
  return first;
}

StatusWord host_moe_pull(HostShmHeap& heap, const HostMoeLayout& lay, const HostMoeShape& s, const int32_t* route,
                         int num_tokens, void* rows, uint64_t epoch, uint64_t timeout_ns) {
  signal_all(heap, FLAG_MOE_Y_READY, epoch);
  StatusWord w = wait_all(heap, FLAG_MOE_Y_READY, epoch, timeout_ns, PHASE_MOE_Y_READY);
  if (w.code != STATUS_OK) return w;
  const int64_t row_bytes = (int64_t)s.hidden * host_dtype_bytes(s.out_dtype);
  uint8_t* dst = static_cast<uint8_t*>(rows);
  at::parallel_for(0, (int64_t)num_tokens * s.topk, grain_for(row_bytes), [&](int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) {
      const int32_t* r = route + 3 * i;
      if (r[0] < 0) {
        std::memset(dst + i * row_bytes, 0, row_bytes);
        continue;
      }
      const uint8_t* src = heap.base(r[0]) + lay.expert_y + ((int64_t)r[1] * s.max_recv + r[2]) * row_bytes;
      std::memcpy(dst + i * row_bytes, src, row_bytes);
    }
  });
  return ok_status();
}

// ---------------------------------------------------------------------------------------
// "dedup" protocol
// ---------------------------------------------------------------------------------------

namespace {

constexpr int kHostMaxChunks = 8;

inline int chunk_begin(int c, int len, int chunks) { return (int)(((int64_t)c * len + chunks - 1) / chunks); }

// destination ranks of token t: owners of its delivered entries, as a bit mask
inline uint32_t owners_of(const int32_t* route, int t, int k, int ws) {
  uint32_t mask = 0;
  for (int kk = 0; kk < k; ++kk) {
    const int32_t* r = route + 2 * ((int64_t)t * k + kk);
    if (r[0] >= 0 && r[0] < ws && r[1] >= 0) mask |= 1u << r[0];
  }
  return mask;
}

}  // namespace

StatusWord host_moe_dedup_dispatch(HostShmHeap& heap, const HostMoeDedupLayout& lay, const HostMoeDedupShape& s,
                                   const void* x, const int32_t* indices, int num_tokens, int32_t* route,
                                   int32_t* expert_num_tokens, uint64_t epoch, uint64_t timeout_ns) {
  const int ws = heap.world_size(), rank = heap.rank();
  const int E = s.num_experts, El = E / ws, k = s.topk, T = num_tokens, n = T * k;
  const int C = std::max(1, std::min(s.chunks, kHostMaxChunks));
  const int64_t row_bytes = (int64_t)s.hidden * host_dtype_bytes(s.in_dtype);
  const int32_t mark = (int32_t)(uint32_t)epoch;
  StatusWord first = ok_status();

  // 1. per-expert counts of this rank, and how it cuts its tokens (call | chunks | tokens), to every rank
  std::vector<int32_t> mine(E, 0);
  for (int i = 0; i < n; ++i) {
    const int e = indices[i];
    if (e < 0 || e >= E) {
      if (first.code == STATUS_OK) first = bad_index(PHASE_MOE_COUNTS, i, epoch, (uint64_t)(int64_t)e);
      continue;
    }
    ++mine[e];
  }
  const uint64_t info = ((epoch & 0xffffffull) << 40) | ((uint64_t)C << 36) | (uint64_t)T;
  for (int i = 1; i <= ws; ++i) {
    const int d = (rank + i) % ws;
    std::memcpy(heap.base(d) + lay.counts + (uint64_t)rank * E * sizeof(int32_t), mine.data(), E * sizeof(int32_t));
    heap.signal(FLAG_MOE_INFO, d, info);
    heap.signal(FLAG_MOE_COUNTS, d, epoch);
  }
  // Everybody's counts for THIS call: every rank has then left its previous call, so nobody still
  // reads the landing rows and records that this call is about to overwrite.
  StatusWord w = wait_all(heap, FLAG_MOE_COUNTS, epoch, timeout_ns, PHASE_MOE_COUNTS);
  if (w.code != STATUS_OK) return w;

  // 2. first slot of this rank inside every expert; rows every local expert holds
  const int32_t* counts = reinterpret_cast<const int32_t*>(heap.base(rank) + lay.counts);
  std::vector<int32_t> next(E);
  for (int e = 0; e < E; ++e) {
    int32_t b = 0;
    for (int src = 0; src < rank; ++src) b += counts[src * E + e];
    next[e] = b;
  }
  for (int el = 0; el < El; ++el) {
    int32_t t = 0;
    for (int src = 0; src < ws; ++src) t += counts[src * E + rank * El + el];
    expert_num_tokens[el] = std::min<int32_t>(t, s.max_recv);
  }

  // 3. final rows in (token, k) order
  for (int i = 0; i < n; ++i) {
    const int e = indices[i];
    int32_t* r = route + 2 * (int64_t)i;
    r[0] = -1, r[1] = -1;
    if (e < 0 || e >= E) continue;
    const int slot = next[e]++;
    r[0] = e / El;
    if (slot >= s.max_recv) {
      if (first.code == STATUS_OK) first = bad_index(PHASE_MOE_DATA, e, epoch, (uint64_t)slot);
      continue;
    }
    r[1] = (e % El) * s.max_recv + slot;
  }

  // 4. chunk by chunk: every token once per destination rank, with its record; then the chunk's flag
  const uint8_t* xb = static_cast<const uint8_t*>(x);
  for (int c = 0; c < C; ++c) {
    const int t0 = chunk_begin(c, T, C), t1 = chunk_begin(c + 1, T, C);
    at::parallel_for(t0, t1, grain_for(row_bytes), [&](int64_t lo, int64_t hi) {
      for (int64_t t = lo; t < hi; ++t) {
        uint32_t mask = owners_of(route, (int)t, k, ws);
        const uint64_t cell = (uint64_t)rank * s.max_tokens + (uint64_t)t;
        while (mask) {
          const int d = __builtin_ctz(mask);
          mask &= mask - 1;
          uint8_t* dst = heap.base(d);
          if (d != rank) std::memcpy(dst + lay.land + cell * row_bytes, xb + t * row_bytes, row_bytes);
          int32_t* rec = reinterpret_cast<int32_t*>(dst + lay.tok_rec) + cell * s.rec_ints;
          for (int kk = 0; kk < k; ++kk) {
            const int32_t* r = route + 2 * (t * k + kk);
            rec[1 + kk] = (r[0] == d) ? r[1] : -1;
            rec[1 + k + kk] = 0;  // the weight arrives with combine
          }
          rec[0] = mark;
        }
      }
    });
    const uint64_t value = (epoch << 8) | (uint64_t)(c + 1);
    for (int i = 1; i <= ws; ++i) heap.signal(FLAG_MOE_DATA, (rank + i) % ws, value);
  }

  // 5. replicate what landed here, chunk by chunk and source by source as the flags come in
  int src_T[kMaxWorldSize], src_C[kMaxWorldSize], c_max = 1;
  for (int src = 0; src < ws; ++src) {
    const uint64_t word = heap.peek(FLAG_MOE_INFO, src);
    const bool fresh = ((word >> 40) & 0xffffffull) == (epoch & 0xffffffull);
    src_T[src] = fresh ? std::min<int>((int)(word & 0xffffffull), s.max_tokens) : 0;
    src_C[src] = fresh ? std::max(1, std::min<int>((int)((word >> 36) & 0xfull), kHostMaxChunks)) : 1;
    c_max = std::max(c_max, src_C[src]);
  }
  const int32_t total_rows = El * s.max_recv;
  const uint8_t* land = heap.base(rank) + lay.land;
  uint8_t* ex = heap.base(rank) + lay.expert_x;
  int32_t* meta = reinterpret_cast<int32_t*>(heap.base(rank) + lay.expert_meta);
  const int32_t* recs = reinterpret_cast<const int32_t*>(heap.base(rank) + lay.tok_rec);
  std::atomic<int64_t> bad_row{-1};
  for (int c = 0; c < c_max; ++c) {
    for (int j = 0; j < ws; ++j) {
      const int src = (rank + j) % ws;  // this rank's own rows first: they are already in place
      const int Cs = src_C[src];
      if (c >= Cs) continue;
      w = heap.wait(FLAG_MOE_DATA, src, (epoch << 8) | (uint64_t)(c + 1), timeout_ns, PHASE_MOE_DATA);
      if (w.code != STATUS_OK) return w;
      const int t0 = chunk_begin(c, src_T[src], Cs), t1 = chunk_begin(c + 1, src_T[src], Cs);
      at::parallel_for(t0, t1, grain_for(row_bytes), [&](int64_t lo, int64_t hi) {
        for (int64_t t = lo; t < hi; ++t) {
          const uint64_t cell = (uint64_t)src * s.max_tokens + (uint64_t)t;
          const int32_t* rec = recs + cell * s.rec_ints;
          if (rec[0] != mark) continue;
          const uint8_t* from = (src == rank) ? xb + t * row_bytes : land + cell * row_bytes;
          for (int kk = 0; kk < k; ++kk) {
            const int32_t row = rec[1 + kk];
            if (row < 0) continue;
            if (row >= total_rows) {
              bad_row.store(row, std::memory_order_relaxed);
              continue;
            }
            std::memcpy(ex + (int64_t)row * row_bytes, from, row_bytes);
            int32_t* m = meta + (int64_t)row * 5;
            m[0] = rank * El + row / s.max_recv;
            m[1] = src;
            m[2] = (int32_t)t;
            m[3] = kk;
            m[4] = 0;
          }
        }
      });
    }
  }
  const int64_t bad = bad_row.load();
  if (bad >= 0 && first.code == STATUS_OK) first = bad_index(PHASE_MOE_DATA, -1, epoch, (uint64_t)bad);
  return first;
}

StatusWord host_moe_dedup_send_weights(HostShmHeap& heap, const HostMoeDedupLayout& lay, const HostMoeDedupShape& s,
                                       const int32_t* route, const float* weights, int num_tokens, uint64_t epoch,
                                       uint64_t timeout_ns) {
  const int ws = heap.world_size(), rank = heap.rank(), k = s.topk;
  for (int t = 0; t < num_tokens; ++t) {
    uint32_t mask = owners_of(route, t, k, ws);
    const uint64_t cell = (uint64_t)rank * s.max_tokens + (uint64_t)t;
    while (mask) {
      const int d = __builtin_ctz(mask);
      mask &= mask - 1;
      float* wrec = reinterpret_cast<float*>(heap.base(d) + lay.tok_rec) + cell * s.rec_ints + 1 + k;
      for (int kk = 0; kk < k; ++kk) {
        const int32_t* r = route + 2 * ((int64_t)t * k + kk);
        wrec[kk] = (r[0] == d && r[1] >= 0) ? weights[(int64_t)t * k + kk] : 0.f;
      }
    }
  }
  signal_all(heap, FLAG_MOE_Y_READY, epoch);
  return wait_all(heap, FLAG_MOE_Y_READY, epoch, timeout_ns, PHASE_MOE_WEIGHTS);
}

StatusWord host_moe_dedup_return(HostShmHeap& heap, uint64_t epoch, uint64_t timeout_ns) {
  signal_all(heap, FLAG_MOE_RET, epoch);
  return wait_all(heap, FLAG_MOE_RET, epoch, timeout_ns, PHASE_MOE_RETURN);
}

StatusWord host_rs_exchange(HostShmHeap& heap, uint64_t stage_offset, const void* partial, int m, int n,
                            int elem_bytes, uint64_t epoch, uint64_t timeout_ns) {
  const int ws = heap.world_size(), rank = heap.rank();
  const int rows = m / ws;
  const int64_t row_bytes = (int64_t)n * elem_bytes;
  const int64_t block_bytes = rows * row_bytes;
  const uint8_t* pb = static_cast<const uint8_t*>(partial);
  // row block d into rank d's slot [src = rank], nearest higher rank first; the own block stays put
  for (int i = 1; i < ws; ++i) {
    const int d = (rank + i) % ws;
    uint8_t* dst = heap.base(d) + stage_offset + (uint64_t)rank * block_bytes;
    const uint8_t* src = pb + (int64_t)d * block_bytes;
    at::parallel_for(0, rows, grain_for(row_bytes), [&](int64_t lo, int64_t hi) {
      std::memcpy(dst + lo * row_bytes, src + lo * row_bytes, (hi - lo) * row_bytes);
    });
    heap.signal(FLAG_RS_DONE, d, epoch);
  }
  heap.signal(FLAG_RS_DONE, rank, epoch);
  return wait_all(heap, FLAG_RS_DONE, epoch, timeout_ns, PHASE_RS_PARTIALS);
}

}  // namespace b200
