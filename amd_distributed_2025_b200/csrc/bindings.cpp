// Python bindings: torch tensors in, raw pointers + current CUDA stream out.
//
// Plays the role of the reference's CPP_WRAPPER / torch::Tensor wrapper pairs
// (all2all/hipv8.py:20-40,229-237), with host-side validation of dtypes, shapes and
// contiguity and launches on the caller's current stream instead of the default stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <memory>
#include <string>
#include <vector>

#include "fp8_gemm.h"
#include "gemm_rs.h"
#include "host_ops.h"
#include "host_shm_heap.h"
#include "mcast_region.h"
#include "moe.h"
#include "status.h"
#include "symm_heap.h"

namespace py = pybind11;
using b200::SymmHeap;

namespace {

void cuda_check(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e));
}

int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kHalf: return 0;
    case at::kBFloat16: return 1;
    case at::kFloat: return 2;
    default: TORCH_CHECK(false, "unsupported dtype ", t, " (expected float16, bfloat16 or float32)");
  }
  return -1;
}

void fill_peer_bases(const SymmHeap& heap, uint64_t* out) {
  for (int r = 0; r < b200::kMaxWorldSize; ++r) out[r] = r < heap.world_size() ? heap.peer_base(r) : 0;
}

py::dict status_to_dict(const b200::StatusWord& w) {
  py::dict d;
  d["code"] = w.code;
  d["phase"] = w.phase;
  d["peer"] = w.peer;
  d["detail"] = w.detail;
  d["epoch"] = w.epoch;
  d["seen"] = w.seen;
  return d;
}

at::Tensor heap_view(SymmHeap& heap, int64_t offset, std::vector<int64_t> shape, at::ScalarType dtype) {
  int64_t numel = 1;
  for (auto s : shape) numel *= s;
  const int64_t nbytes = numel * (int64_t)c10::elementSize(dtype);
  TORCH_CHECK(offset >= 0 && (uint64_t)(offset + nbytes) <= heap.bytes(), "heap view [", offset, ", ",
              offset + nbytes, ") exceeds the slab of ", heap.bytes(), " bytes");
  auto opts = at::TensorOptions().dtype(dtype).device(at::kCUDA, heap.device());
  return at::from_blob(static_cast<uint8_t*>(heap.local_base()) + offset, shape, opts);
}

// ----------------------------------------------------------------------------- MoE ----

void moe_dispatch(SymmHeap& heap, const at::Tensor& x, const at::Tensor& indices, int64_t num_experts,
                  int64_t max_recv, int64_t off_counts, int64_t off_expert_x, int64_t off_expert_meta,
                  at::Tensor blk_hist, at::Tensor local_rank, at::Tensor route, at::Tensor expert_num_tokens,
                  int64_t epoch, int64_t timeout_ns) {
  TORCH_CHECK(heap.peers_open(), "symmetric heap: peers are not mapped yet");
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous(), "x must be a contiguous [T, H] CUDA tensor");
  TORCH_CHECK(indices.is_cuda() && indices.dim() == 2 && indices.is_contiguous() && indices.scalar_type() == at::kInt,
              "indices must be a contiguous [T, k] int32 CUDA tensor");
  TORCH_CHECK(indices.size(0) == x.size(0), "x and indices disagree on the token count");
  TORCH_CHECK(x.get_device() == heap.device(), "x is not on the heap's device");
  const int ws = heap.world_size();
  TORCH_CHECK(num_experts % ws == 0, "num_experts must be divisible by world_size");
  const int64_t T = x.size(0), k = indices.size(1), n = T * k;
  const int64_t e_local = num_experts / ws;
  TORCH_CHECK(e_local * max_recv < (1ll << 31), "expert buffer has too many rows for 32-bit row ids");
  TORCH_CHECK(n < (1ll << 31), "too many (token, k) entries");

  c10::cuda::CUDAGuard guard(heap.device());
  const int max_blocks = b200::moe_dispatch_max_blocks(heap.device());
  int64_t chunk = (n + max_blocks - 1) / max_blocks;
  if (chunk < 32) chunk = 32;
  const int64_t count_blocks = (n + chunk - 1) / chunk;
  int grid = max_blocks;
  // Small problems: fewer CTAs make the in-GPU barrier cheaper; keep enough warps (8 per
  // CTA) to move all rows at once and at least one CTA per rank for the count broadcast.
  const int64_t want = std::max<int64_t>(std::max<int64_t>(count_blocks, (n + 7) / 8), std::min<int64_t>(ws, max_blocks));
  if (want < grid) grid = (int)std::max<int64_t>(want, 1);

  TORCH_CHECK(blk_hist.scalar_type() == at::kInt && blk_hist.is_contiguous() &&
                  blk_hist.numel() >= std::max<int64_t>(count_blocks, 1) * num_experts,
              "blk_hist scratch too small");
  TORCH_CHECK(local_rank.scalar_type() == at::kInt && local_rank.is_contiguous() && local_rank.numel() >= n,
              "local_rank scratch too small");
  TORCH_CHECK(route.scalar_type() == at::kInt && route.is_contiguous() && route.numel() >= 2 * n,
              "route must hold 2 int32 per (token, k) entry");
  TORCH_CHECK(expert_num_tokens.scalar_type() == at::kInt && expert_num_tokens.numel() >= e_local,
              "expert_num_tokens too small");

  b200::MoeDispatchParams p;
  p.x = x.data_ptr();
  p.indices = indices.data_ptr<int32_t>();
  p.num_tokens = (int32_t)T;
  p.k = (int32_t)k;
  p.num_experts = (int32_t)num_experts;
  p.num_local_experts = (int32_t)e_local;
  p.world_size = ws;
  p.rank = heap.rank();
  p.max_recv = (int32_t)max_recv;
  p.row_bytes = (uint32_t)(x.size(1) * x.element_size());
  p.epoch = (uint64_t)epoch;
  p.timeout_ns = (uint64_t)timeout_ns;
  fill_peer_bases(heap, p.peer_base);
  p.layout.off_counts = (uint64_t)off_counts;
  p.layout.off_expert_x = (uint64_t)off_expert_x;
  p.layout.off_expert_meta = (uint64_t)off_expert_meta;
  p.layout.off_expert_y = 0;
  p.blk_hist = blk_hist.data_ptr<int32_t>();
  p.local_rank = local_rank.data_ptr<int32_t>();
  p.route = reinterpret_cast<int2*>(route.data_ptr<int32_t>());
  p.expert_num_tokens = expert_num_tokens.data_ptr<int32_t>();
  p.sync_counters = heap.sync_counters();
  p.status = heap.status_device();
  p.count_blocks = (int32_t)count_blocks;
  p.chunk = (int32_t)chunk;
  if (b200::moe_dispatch_small_applies((int)n, (int)num_experts)) {
    // one warp per entry, at least one CTA per rank for the count broadcast, any number of CTAs
    const int small_grid = (int)std::max<int64_t>(std::min<int64_t>((n + 7) / 8, 2 * max_blocks), std::max(ws, 1));
    cuda_check(b200::launch_moe_dispatch_small(p, small_grid, at::cuda::getCurrentCUDAStream()), "moe_dispatch launch");
    return;
  }
  cuda_check(b200::launch_moe_dispatch(p, grid, at::cuda::getCurrentCUDAStream()), "moe_dispatch launch");
}

void moe_expert_scale(const at::Tensor& expert_x, at::Tensor expert_y, const at::Tensor& expert_num_tokens,
                      double scale) {
  TORCH_CHECK(expert_x.dim() == 3 && expert_y.sizes() == expert_x.sizes(), "expert_x / expert_y shapes differ");
  TORCH_CHECK(expert_x.is_contiguous() && expert_y.is_contiguous(), "expert buffers must be contiguous");
  c10::cuda::CUDAGuard guard(expert_x.device());
  cuda_check(b200::launch_moe_expert_scale(expert_x.data_ptr(), expert_y.data_ptr(),
                                           expert_num_tokens.data_ptr<int32_t>(), (int)expert_x.size(0),
                                           (int)expert_x.size(1), (int)expert_x.size(2),
                                           dtype_code(expert_x.scalar_type()), dtype_code(expert_y.scalar_type()),
                                           (float)scale, at::cuda::getCurrentCUDAStream()),
             "moe_expert_scale launch");
}

void moe_combine(SymmHeap& heap, at::Tensor out, const at::Tensor& weights, const at::Tensor& route,
                 int64_t num_tokens, int64_t max_recv, int64_t off_expert_y, int64_t epoch, int64_t timeout_ns) {
  TORCH_CHECK(heap.peers_open(), "symmetric heap: peers are not mapped yet");
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.is_contiguous(), "out must be a contiguous [T, H] CUDA tensor");
  TORCH_CHECK(weights.scalar_type() == at::kFloat && weights.is_contiguous() && weights.dim() == 2,
              "weights must be contiguous fp32 [T, k]");
  TORCH_CHECK(out.size(0) >= num_tokens && weights.size(0) >= num_tokens, "out/weights have fewer rows than tokens");
  const int64_t k = weights.size(1);
  TORCH_CHECK(route.scalar_type() == at::kInt && route.numel() >= 2 * num_tokens * k, "route too small");
  c10::cuda::CUDAGuard guard(heap.device());
  b200::MoeCombineParams p;
  p.out = out.data_ptr();
  p.weights = weights.data_ptr<float>();
  p.route = reinterpret_cast<const int2*>(route.data_ptr<int32_t>());
  p.num_tokens = (int32_t)num_tokens;
  p.k = (int32_t)k;
  p.hidden = (int32_t)out.size(1);
  p.world_size = heap.world_size();
  p.rank = heap.rank();
  p.max_recv = (int32_t)max_recv;
  p.dtype = dtype_code(out.scalar_type());
  p.epoch = (uint64_t)epoch;
  p.timeout_ns = (uint64_t)timeout_ns;
  fill_peer_bases(heap, p.peer_base);
  p.off_expert_y = (uint64_t)off_expert_y;
  p.status = heap.status_device();
  cuda_check(b200::launch_moe_combine(p, at::cuda::getCurrentCUDAStream()), "moe_combine launch");
}

// The whole task pipeline in one call: dispatch, the per-rank scale that stands in for the
// expert computation (all2all/reference.py:262), combine.  Three launches, no host work in
// between, so short problems are not bound by the Python call overhead.
void moe_forward(SymmHeap& heap, const at::Tensor& x, const at::Tensor& indices, const at::Tensor& weights,
                 at::Tensor out, int64_t num_experts, int64_t max_recv, int64_t off_counts, int64_t off_expert_x,
                 int64_t off_expert_meta, int64_t off_expert_y, at::Tensor expert_x, at::Tensor expert_y,
                 at::Tensor blk_hist, at::Tensor local_rank, at::Tensor route, at::Tensor expert_num_tokens,
                 double scale, int64_t dispatch_epoch, int64_t combine_epoch, int64_t timeout_ns) {
  moe_dispatch(heap, x, indices, num_experts, max_recv, off_counts, off_expert_x, off_expert_meta, blk_hist,
               local_rank, route, expert_num_tokens, dispatch_epoch, timeout_ns);
  moe_expert_scale(expert_x, expert_y, expert_num_tokens, scale);
  moe_combine(heap, out, weights, route, x.size(0), max_recv, off_expert_y, combine_epoch, timeout_ns);
}


// ----------------------------------------------------- MoE, de-duplicating protocol ----
// One object per layer keeps everything that does not change between calls (heap, offsets,
// scratch, grid sizes, epochs), so a call converts three or four tensors and launches.
class MoeDedupEngine {
 public:
  MoeDedupEngine(std::shared_ptr<SymmHeap> heap, int64_t num_experts, int64_t topk, int64_t hidden, int64_t max_tokens,
                 int64_t max_recv, at::ScalarType dtype, bool partial_fp32, std::vector<int64_t> offsets,
                 at::Tensor expert_y, at::Tensor blk_hist, at::Tensor route, at::Tensor expert_num_tokens,
                 int64_t timeout_ns)
      : heap_(std::move(heap)), E_(num_experts), k_(topk), H_(hidden), max_tokens_(max_tokens), max_recv_(max_recv),
        dtype_(dtype), partial_fp32_(partial_fp32), expert_y_(std::move(expert_y)), blk_hist_(std::move(blk_hist)),
        route_(std::move(route)), expert_num_tokens_(std::move(expert_num_tokens)), timeout_ns_(timeout_ns) {
    TORCH_CHECK(heap_->peers_open(), "symmetric heap: peers are not mapped yet");
    const int ws = heap_->world_size();
    TORCH_CHECK(E_ > 0 && E_ % ws == 0, "num_experts must be divisible by world_size");
    TORCH_CHECK(k_ >= 1 && k_ <= 15, "experts_per_token must be in 1..15 (one 32-lane store per token record)");
    TORCH_CHECK(offsets.size() == 7, "expected 7 region offsets");
    El_ = E_ / ws;
    TORCH_CHECK(El_ * max_recv_ < (1ll << 31), "expert buffer has too many rows for 32-bit row ids");
    lay_.off_counts = (uint64_t)offsets[0];
    lay_.off_expert_x = (uint64_t)offsets[1];
    lay_.off_expert_meta = (uint64_t)offsets[2];
    lay_.off_expert_y = (uint64_t)offsets[3];
    lay_.off_land = (uint64_t)offsets[4];
    lay_.off_tok_rec = (uint64_t)offsets[5];
    lay_.off_ret = (uint64_t)offsets[6];
    rec_ints_ = (int)((1 + 2 * k_ + 3) / 4 * 4);
    elem_ = (int64_t)c10::elementSize(dtype_);
    dtype_code_ = dtype_code(dtype_);
    TORCH_CHECK(route_.scalar_type() == at::kInt && route_.is_contiguous() && route_.numel() >= 2 * max_tokens_ * k_,
                "route must hold 2 int32 per (token, k) entry");
    TORCH_CHECK(expert_num_tokens_.scalar_type() == at::kInt && expert_num_tokens_.numel() >= El_, "expert_num_tokens too small");
    TORCH_CHECK(expert_y_.is_contiguous() && expert_y_.scalar_type() == dtype_ && expert_y_.numel() == El_ * max_recv_ * H_,
                "expert_y must be a contiguous [E_local, max_recv, hidden] tensor of the layer's dtype");
    c10::cuda::CUDAGuard guard(heap_->device());
    combine_blocks_ = b200::moe_dedup_combine_max_blocks(heap_->device());
    TORCH_CHECK(blk_hist_.scalar_type() == at::kInt && blk_hist_.is_contiguous(), "blk_hist must be contiguous int32");
  }

  int64_t chunks = 4;        // chunks of a large dispatch (1 = all rows under one flag)
  int64_t chunk_min_ranks = 4;  // chunking starts at this world size ...
  int64_t chunk_min_bytes = 8 << 20;  // ... and at this many bytes of token rows per rank
  bool bulk_landing = true;  // rows cross NVLink as bulk copies through shared memory (else 16-byte stores)
  int64_t dispatch_epoch() const { return dispatch_epoch_; }
  int64_t combine_epoch() const { return combine_epoch_; }
  void set_timeout_ns(int64_t t) { timeout_ns_ = t; }
  void set_trace(const c10::optional<at::Tensor>& dispatch_trace, const c10::optional<at::Tensor>& combine_trace) {
    trace_d_ = check_trace(dispatch_trace);
    trace_c_ = check_trace(combine_trace);
  }

  // dispatch / combine / forward return 0 after launching, or the code of a failure that an earlier
  // kernel recorded (nothing is launched then; the caller turns the record into an exception).
  int dispatch(const at::Tensor& x, const at::Tensor& indices, const c10::optional<at::Tensor>& weights,
               bool fuse_scale, double scale) {
    if (const uint32_t code = heap_->status_host().code) return (int)code;
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && x.scalar_type() == dtype_ && x.size(1) == H_,
                "x must be a contiguous [T, hidden] CUDA tensor of the layer's dtype");
    TORCH_CHECK(indices.is_cuda() && indices.dim() == 2 && indices.is_contiguous() && indices.scalar_type() == at::kInt &&
                    indices.size(0) == x.size(0) && indices.size(1) == k_,
                "indices must be a contiguous [T, k] int32 CUDA tensor");
    TORCH_CHECK(x.get_device() == heap_->device(), "x is not on the heap's device");
    const int64_t T = x.size(0);
    TORCH_CHECK(T <= max_tokens_, T, " tokens exceed max_num_tokens=", max_tokens_);
    const float* wptr = nullptr;
    if (weights.has_value() && weights->defined()) {
      TORCH_CHECK(weights->is_cuda() && weights->scalar_type() == at::kFloat && weights->is_contiguous() &&
                      weights->dim() == 2 && weights->size(0) == T && weights->size(1) == k_,
                  "weights must be contiguous fp32 [T, k]");
      wptr = weights->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(heap_->device());
    const int ws = heap_->world_size();
    const int n = (int)(T * k_);
    const int bulk = (bulk_landing && ws > 1 && (H_ * elem_) % 16 == 0) ? 1 : 0;
    const int max_blocks = b200::moe_dedup_dispatch_max_blocks(heap_->device(), (int)E_, n, bulk);
    TORCH_CHECK(blk_hist_.numel() >= (int64_t)max_blocks * E_, "blk_hist scratch too small");
    b200::MoeDedupDispatchParams p;
    p.x = x.data_ptr();
    p.indices = indices.data_ptr<int32_t>();
    p.weights = wptr;
    p.num_tokens = (int32_t)T;
    p.k = (int32_t)k_;
    p.num_experts = (int32_t)E_;
    p.num_local_experts = (int32_t)El_;
    p.world_size = ws;
    p.rank = heap_->rank();
    p.max_recv = (int32_t)max_recv_;
    p.max_tokens = (int32_t)max_tokens_;
    p.rec_ints = rec_ints_;
    p.dtype = dtype_code_;
    p.row_bytes = (uint32_t)(H_ * elem_);
    // Large transfers between GPUs go in chunks with their own "delivered" flags, so that the owners
    // replicate one chunk while the next is still crossing the links.
    const bool small = b200::moe_dedup_is_small(n, (int)E_);
    // (pays when a rank's inbound link, not its memory, sets the pace: measured a loss on 2 ranks)
    p.chunks = (!small && ws >= chunk_min_ranks && T * H_ * elem_ >= chunk_min_bytes) ? (int)chunks : 1;
    p.pieces = pieces_for((int)T, max_blocks, 1);
    // Replication goes source by source, so one loop has (tokens of one source's chunk) x pieces items.
    // Measured: on 8 ranks one piece per row (a hot owner's 1024 live rows per loop already fill the
    // grid's warps once, and every further piece costs another dependent record load); on fewer
    // ranks the finer split, which evens out the warps' shares.
    p.rep_pieces = pieces_for((int)std::max<int64_t>(T / p.chunks, 1), max_blocks, ws >= 8 ? 12 : 32);
    p.bulk_landing = bulk;
    p.fuse_scale = fuse_scale ? 1 : 0;
    p.scale = (float)scale;
    p.epoch = (uint64_t)(++dispatch_epoch_);
    p.timeout_ns = (uint64_t)timeout_ns_;
    fill_peer_bases(*heap_, p.peer_base);
    p.layout = lay_;
    p.expert_y = expert_y_.data_ptr();
    p.blk_hist = blk_hist_.data_ptr<int32_t>();
    p.route = reinterpret_cast<int2*>(route_.data_ptr<int32_t>());
    p.expert_num_tokens = expert_num_tokens_.data_ptr<int32_t>();
    p.sync_counters = heap_->sync_counters();
    p.status = heap_->status_device();
    p.trace = trace_d_;
    // enough warps for every (source, token, piece) of the replication pass, never more CTAs than fit at once
    const int64_t want = ((int64_t)ws * std::max<int64_t>(T, 1) * p.pieces + 7) / 8;
    const int grid = (int)std::max<int64_t>(std::min<int64_t>(max_blocks, want), 1);
    weights_sent_ = wptr != nullptr;
    num_tokens_ = (int)T;
    cuda_check(b200::launch_moe_dedup_dispatch(p, grid, at::cuda::getCurrentCUDAStream()), "moe_dedup_dispatch launch");
    return 0;
  }

  int combine(at::Tensor out, const at::Tensor& weights, const c10::optional<at::Tensor>& expert_y) {
    if (const uint32_t code = heap_->status_host().code) return (int)code;
    const int64_t T = num_tokens_;
    TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.is_contiguous() && out.scalar_type() == dtype_ &&
                    out.size(0) >= T && out.size(1) == H_,
                "out must be a contiguous [>= T, hidden] CUDA tensor of the layer's dtype");
    TORCH_CHECK(weights.is_cuda() && weights.scalar_type() == at::kFloat && weights.is_contiguous() && weights.dim() == 2 &&
                    weights.size(0) >= T && weights.size(1) == k_,
                "weights must be contiguous fp32 [T, k]");
    const void* ey = expert_y_.data_ptr();
    if (expert_y.has_value() && expert_y->defined()) {
      TORCH_CHECK(expert_y->is_cuda() && expert_y->is_contiguous() && expert_y->scalar_type() == dtype_ &&
                      expert_y->numel() == El_ * max_recv_ * H_,
                  "expert_y does not have the dispatch layout / dtype");
      ey = expert_y->data_ptr();
    }
    c10::cuda::CUDAGuard guard(heap_->device());
    const int ws = heap_->world_size();
    b200::MoeDedupCombineParams p;
    p.out = out.data_ptr();
    p.weights = weights.data_ptr<float>();
    p.route = reinterpret_cast<const int2*>(route_.data_ptr<int32_t>());
    p.expert_y = ey;
    p.num_tokens = (int32_t)T;
    p.k = (int32_t)k_;
    p.hidden = (int32_t)H_;
    p.num_local_experts = (int32_t)El_;
    p.world_size = ws;
    p.rank = heap_->rank();
    p.max_recv = (int32_t)max_recv_;
    p.max_tokens = (int32_t)max_tokens_;
    p.rec_ints = rec_ints_;
    p.dtype = dtype_code_;
    p.partial_fp32 = partial_fp32_ ? 1 : 0;
    p.weights_sent = weights_sent_ ? 1 : 0;
    p.pieces = pieces_for((int)T, combine_blocks_, 4);
    p.epoch = (uint64_t)(++combine_epoch_);
    p.dispatch_epoch = (uint64_t)dispatch_epoch_;
    p.timeout_ns = (uint64_t)timeout_ns_;
    fill_peer_bases(*heap_, p.peer_base);
    p.layout = lay_;
    p.sync_counters = heap_->sync_counters();
    p.status = heap_->status_device();
    p.trace = trace_c_;
    const int64_t want = ((int64_t)ws * std::max<int64_t>(T, 1) * p.pieces + 7) / 8;
    const int grid = (int)std::max<int64_t>(std::min<int64_t>(combine_blocks_, want), 1);
    cuda_check(b200::launch_moe_dedup_combine(p, grid, at::cuda::getCurrentCUDAStream()), "moe_dedup_combine launch");
    // A further combine of the same dispatch (other weights, another expert output) sends its own
    // weights: that exchange is also the rendezvous which keeps an owner from pushing new partial
    // rows while a source still adds up the previous ones.
    weights_sent_ = false;
    return 0;
  }

  // dispatch (carrying the weights, applying expert_y = expert_x * scale on the way) + combine
  int forward(const at::Tensor& x, const at::Tensor& indices, const at::Tensor& weights, at::Tensor out, double scale) {
    if (const int rc = dispatch(x, indices, weights, true, scale)) return rc;
    return combine(out, weights, c10::nullopt);
  }

 private:
  uint64_t* check_trace(const c10::optional<at::Tensor>& t) {
    if (!t.has_value() || !t->defined()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kLong && t->is_contiguous() && t->numel() >= 8,
                "trace must be a contiguous int64 CUDA tensor with at least 8 elements");
    keep_.push_back(*t);
    return reinterpret_cast<uint64_t*>(t->data_ptr<int64_t>());
  }
  // A row is split over several warps so that there are about `per_warp` (row, piece) items for
  // every warp of the grid: one when a row's latency matters (decode), a dozen when the point is
  // that all warps get nearly equal shares.  Power of two, at most 8, at least 1 KiB per piece.
  int pieces_for(int tokens, int blocks, int per_warp) const {
    const int64_t row_bytes = H_ * elem_;
    if (row_bytes % 16 != 0) return 1;
    const int nv = (int)(row_bytes / 16);
    const int64_t want = ((int64_t)per_warp * blocks * 8) / std::max<int64_t>((int64_t)tokens * heap_->world_size(), 1);
    int pcs = 1;
    while (pcs < 8 && pcs * 2 <= want && nv / (pcs * 2) >= 64) pcs *= 2;
    return pcs;
  }

  std::shared_ptr<SymmHeap> heap_;
  int64_t E_, k_, H_, max_tokens_, max_recv_, El_ = 0, elem_ = 2;
  at::ScalarType dtype_;
  int dtype_code_ = 0;
  int rec_ints_ = 4;
  bool partial_fp32_;
  b200::MoeDedupLayout lay_;
  at::Tensor expert_y_, blk_hist_, route_, expert_num_tokens_;
  int64_t timeout_ns_;
  int64_t dispatch_epoch_ = 0, combine_epoch_ = 0;
  int combine_blocks_ = 1;
  bool weights_sent_ = false;
  int num_tokens_ = 0;
  uint64_t* trace_d_ = nullptr;
  uint64_t* trace_c_ = nullptr;
  std::vector<at::Tensor> keep_;
};

// ------------------------------------------------------------------------- GEMM-RS ----

void gemm_rs(SymmHeap& heap, const at::Tensor& a, const at::Tensor& w, const c10::optional<at::Tensor>& bias,
             at::Tensor out, double bias_scale, bool bias_at_source, int64_t off_stage, int64_t off_counters, int64_t epoch,
             int64_t timeout_ns, int64_t max_ctas, int64_t block_n, int64_t cta_pair, int64_t splits,
             const c10::optional<at::Tensor>& trace, int64_t debug, bool fuse_own, bool tma_store, bool force_staged,
             bool checked, int64_t stage_capacity) {
  TORCH_CHECK(heap.peers_open(), "symmetric heap: peers are not mapped yet");
  TORCH_CHECK(a.is_cuda() && w.is_cuda() && a.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16,
              "input and weight must be bf16 CUDA tensors");
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && a.size(1) == w.size(1), "input [M, K] and weight [N, K] disagree on K");
  TORCH_CHECK(a.is_contiguous() && w.is_contiguous() && out.is_contiguous(), "operands must be contiguous");
  const int ws = heap.world_size();
  const int64_t M = a.size(0), N = w.size(0), K = a.size(1);
  TORCH_CHECK(M % ws == 0, "M must be divisible by world_size");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.size(0) == M / ws && out.size(1) == N, "out must be bf16 [M/ws, N]");
  TORCH_CHECK(K % 8 == 0, "K per rank must be a multiple of 8 (16-byte rows for TMA)");
  TORCH_CHECK(N % 8 == 0, "N must be a multiple of 8 (16-byte vector epilogue)");
  const void* bias_ptr = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == N && bias->is_contiguous(), "bias must be bf16 [N]");
    bias_ptr = bias->data_ptr();
  }
  c10::cuda::CUDAGuard guard(heap.device());
  b200::GemmRsArgs g;
  g.a = a.data_ptr();
  g.w = w.data_ptr();
  g.bias = bias_ptr;
  g.out = out.data_ptr();
  g.M = (int)M;
  g.N = (int)N;
  g.K = (int)K;
  g.world_size = ws;
  g.rank = heap.rank();
  g.bias_scale = (float)bias_scale;
  g.bias_at_source = bias_at_source ? 1 : 0;
  fill_peer_bases(heap, g.peer_base);
  g.off_stage = (uint64_t)off_stage;
  g.off_counters = (uint64_t)off_counters;
  g.epoch = (uint64_t)epoch;
  g.timeout_ns = (uint64_t)timeout_ns;
  g.status = heap.status_device();
  g.sync_counters = heap.sync_counters() + 8;
  g.max_ctas = (int)max_ctas;
  g.block_n = (int)block_n;
  g.cta_pair = (int)cta_pair;
  g.splits = (int)splits;
  g.trace = nullptr;
  g.debug = (int)debug;
  g.fuse_own = fuse_own ? 1 : 0;
  g.tma_store = tma_store ? 1 : 0;
  g.force_staged = force_staged ? 1 : 0;
  g.checked = checked ? 1 : 0;
  g.stage_capacity = (uint64_t)stage_capacity;
  g.nvls_local = 0;
  g.nvls_mc = 0;
  if (trace.has_value() && trace->defined()) {
    TORCH_CHECK(trace->scalar_type() == at::kLong && trace->is_contiguous() && trace->numel() >= 8 * 160,
                "trace must be a contiguous int64 tensor with at least 1280 elements");
    g.trace = reinterpret_cast<uint64_t*>(trace->data_ptr<int64_t>());
  }
  cuda_check(b200::launch_gemm_rs(g, at::cuda::getCurrentCUDAStream()), "gemm_rs launch");
}


// One object per GEMM-RS workspace: offsets of both parities, the call number and the knobs
// live here, so a call converts four tensors, looks its plan up and launches.
class GemmRsEngine {
 public:
  GemmRsEngine(std::shared_ptr<SymmHeap> heap, std::vector<int64_t> stage_offsets, std::vector<int64_t> counter_offsets,
               int64_t stage_bytes, int64_t counter_bytes, int64_t timeout_ns)
      : heap_(std::move(heap)), stage_bytes_(stage_bytes), counter_bytes_(counter_bytes), timeout_ns_(timeout_ns) {
    TORCH_CHECK(stage_offsets.size() == 2 && counter_offsets.size() == 2, "two parities of staging and counters");
    for (int i = 0; i < 2; ++i) {
      off_stage_[i] = (uint64_t)stage_offsets[i];
      off_counters_[i] = (uint64_t)counter_offsets[i];
    }
  }

  // knobs (0 / -1 = chosen from the shape); see GemmRsArgs
  int64_t max_ctas = 0, block_n = 0, cta_pair = -1, splits = 0, debug = 0;
  int64_t fuse_own = -1;  // -1: fused up to 4 ranks
  bool tma_store = true, force_staged = false, checked = false;

  int64_t epoch() const { return epoch_; }
  void restart_epochs() { epoch_ = 0; }
  // NVLS mode: stage in a multicast region that holds two parities of bf16 [M][N]; nullptr = back to peer stores
  void set_mcast(std::shared_ptr<b200::McastRegion> region) {
    TORCH_CHECK(!region || (region->mapped() && (int64_t)region->bytes() >= 2 * stage_bytes_),
                "the multicast region must be mapped and hold two staging parities");
    mcast_ = std::move(region);
  }
  bool nvls() const { return (bool)mcast_; }
  void set_trace(const c10::optional<at::Tensor>& trace) {
    trace_ = nullptr;
    trace_keep_ = at::Tensor();
    if (trace.has_value() && trace->defined()) {
      TORCH_CHECK(trace->is_cuda() && trace->scalar_type() == at::kLong && trace->is_contiguous() && trace->numel() >= 8 * 160,
                  "trace must be a contiguous int64 CUDA tensor with at least 1280 elements");
      trace_keep_ = *trace;
      trace_ = reinterpret_cast<uint64_t*>(trace->data_ptr<int64_t>());
    }
  }

  py::dict plan(int64_t M, int64_t N, int64_t K) {
    c10::cuda::CUDAGuard guard(heap_->device());
    const b200::GemmRsPlan p = b200::gemm_rs_plan((int)M, (int)N, (int)K, heap_->world_size(), (int)block_n, (int)cta_pair, (int)splits);
    py::dict d;
    d["block_n"] = p.block_n;
    d["cta_pair"] = p.cta_pair;
    d["splits"] = p.splits;
    d["stage_bytes"] = (int64_t)p.stage_bytes;
    d["counter_bytes"] = (int64_t)p.counter_bytes;
    return d;
  }

  // Returns 0 after a launch, or the code of a failure that an earlier kernel recorded (nothing is
  // launched then; the caller turns the record into an exception).
  int run(const at::Tensor& a, const at::Tensor& w, const c10::optional<at::Tensor>& bias, at::Tensor out,
          bool bias_at_source, double bias_scale) {
    TORCH_CHECK(heap_->peers_open(), "symmetric heap: peers are not mapped yet");
    if (const uint32_t code = heap_->status_host().code) return (int)code;
    TORCH_CHECK(a.is_cuda() && w.is_cuda() && a.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16,
                "input and weight must be bf16 CUDA tensors");
    TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && a.size(1) == w.size(1), "input [M, K] and weight [N, K] disagree on K");
    TORCH_CHECK(a.is_contiguous() && w.is_contiguous() && out.is_contiguous(), "operands must be contiguous");
    const int ws = heap_->world_size();
    const int64_t M = a.size(0), N = w.size(0), K = a.size(1);
    TORCH_CHECK(M % ws == 0, "M must be divisible by world_size");
    TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.size(0) == M / ws && out.size(1) == N, "out must be bf16 [M/ws, N]");
    TORCH_CHECK(K % 8 == 0, "K per rank must be a multiple of 8 (16-byte rows for TMA)");
    TORCH_CHECK(N % 8 == 0, "N must be a multiple of 8 (16-byte vector epilogue)");
    const void* bias_ptr = nullptr;
    if (bias.has_value() && bias->defined()) {
      TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == N && bias->is_contiguous(), "bias must be bf16 [N]");
      bias_ptr = bias->data_ptr();
    }
    c10::cuda::CUDAGuard guard(heap_->device());
    const b200::GemmRsPlan plan = cached_plan((int)M, (int)N, (int)K);
    TORCH_CHECK((int64_t)plan.stage_bytes <= stage_bytes_ && (int64_t)plan.counter_bytes <= counter_bytes_, "problem ", M, "x",
                N, "x", K, " needs ", plan.stage_bytes, " staging bytes, the workspace has ", stage_bytes_);
    b200::GemmRsArgs g;
    g.a = a.data_ptr();
    g.w = w.data_ptr();
    g.bias = bias_ptr;
    g.out = out.data_ptr();
    g.M = (int)M;
    g.N = (int)N;
    g.K = (int)K;
    g.world_size = ws;
    g.rank = heap_->rank();
    g.bias_scale = (float)bias_scale;
    g.bias_at_source = bias_at_source ? 1 : 0;
    fill_peer_bases(*heap_, g.peer_base);
    const int64_t epoch = ++epoch_;
    const int parity = (int)(epoch & 1);
    g.off_stage = off_stage_[parity];
    g.off_counters = off_counters_[parity];
    g.epoch = (uint64_t)epoch;
    g.timeout_ns = (uint64_t)timeout_ns_;
    g.status = heap_->status_device();
    g.sync_counters = heap_->sync_counters() + 8;
    g.max_ctas = (int)max_ctas;
    g.block_n = plan.block_n;
    g.cta_pair = plan.cta_pair;
    g.splits = plan.splits;
    g.trace = trace_;
    g.debug = (int)debug;
    g.fuse_own = fuse_own < 0 ? (ws <= 4 ? 1 : 0) : (fuse_own != 0 ? 1 : 0);
    g.tma_store = tma_store ? 1 : 0;
    g.force_staged = force_staged ? 1 : 0;
    g.checked = checked ? 1 : 0;
    g.stage_capacity = (uint64_t)stage_bytes_;
    g.nvls_local = 0;
    g.nvls_mc = 0;
    if (mcast_ && plan.splits == 1 && ws > 1 && !force_staged) {
      const uint64_t off = (uint64_t)parity * (uint64_t)stage_bytes_;
      g.nvls_local = reinterpret_cast<uint64_t>(mcast_->local_ptr()) + off;
      g.nvls_mc = reinterpret_cast<uint64_t>(mcast_->mc_ptr()) + off;
    }
    cuda_check(b200::launch_gemm_rs(g, at::cuda::getCurrentCUDAStream()), "gemm_rs launch");
    return 0;
  }

 private:
  b200::GemmRsPlan cached_plan(int M, int N, int K) {
    for (const auto& e : plans_)
      if (e.M == M && e.N == N && e.K == K && e.block_n == block_n && e.cta_pair == cta_pair && e.splits == splits) return e.plan;
    PlanEntry e{M, N, K, block_n, cta_pair, splits,
                b200::gemm_rs_plan(M, N, K, heap_->world_size(), (int)block_n, (int)cta_pair, (int)splits)};
    if (plans_.size() >= 32) plans_.erase(plans_.begin());
    plans_.push_back(e);
    return e.plan;
  }
  struct PlanEntry {
    int M, N, K;
    int64_t block_n, cta_pair, splits;
    b200::GemmRsPlan plan;
  };
  std::shared_ptr<SymmHeap> heap_;
  uint64_t off_stage_[2], off_counters_[2];
  int64_t stage_bytes_, counter_bytes_, timeout_ns_;
  int64_t epoch_ = 0;
  uint64_t* trace_ = nullptr;
  at::Tensor trace_keep_;
  std::vector<PlanEntry> plans_;
  std::shared_ptr<b200::McastRegion> mcast_;
};

// ------------------------------------------------------------------------ fp8 GEMM ----

void fp8_gemm(const at::Tensor& a, const at::Tensor& b, const at::Tensor& a_scale, const at::Tensor& b_scale,
              at::Tensor c, at::Tensor error_flag, int64_t timeout_ns) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1),
              "a [M, K] and b [N, K] must be CUDA matrices with equal K");
  TORCH_CHECK(a.scalar_type() == at::kFloat8_e4m3fn && b.scalar_type() == at::kFloat8_e4m3fn, "a and b must be float8_e4m3fn");
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous(), "a and b must be row-major (K contiguous)");
  const int64_t M = a.size(0), N = b.size(0), K = a.size(1);
  const int64_t kb = (K + 127) / 128, nb = (N + 127) / 128;
  TORCH_CHECK(a_scale.scalar_type() == at::kFloat && a_scale.dim() == 2 && a_scale.size(0) == M && a_scale.size(1) == kb,
              "a_scale must be fp32 [M, ceil(K/128)]");
  TORCH_CHECK(b_scale.scalar_type() == at::kFloat && b_scale.dim() == 2 && b_scale.size(0) == nb && b_scale.size(1) == kb,
              "b_scale must be fp32 [ceil(N/128), ceil(K/128)]");
  TORCH_CHECK(c.scalar_type() == at::kBFloat16 && c.is_contiguous() && c.size(0) == M && c.size(1) == N, "c must be bf16 [M, N]");
  TORCH_CHECK(K % 16 == 0, "K must be a multiple of 16");
  TORCH_CHECK(error_flag.scalar_type() == at::kInt && error_flag.numel() >= 1, "error_flag must be an int32 tensor");
  c10::cuda::CUDAGuard guard(a.device());
  b200::Fp8GemmArgs g;
  g.a = a.data_ptr();
  g.b = b.data_ptr();
  g.a_scale = a_scale.data_ptr<float>();
  g.b_scale = b_scale.data_ptr<float>();
  g.c = c.data_ptr();
  g.M = (int)M;
  g.N = (int)N;
  g.K = (int)K;
  g.as_stride_m = a_scale.stride(0);
  g.as_stride_k = a_scale.stride(1);
  g.bs_stride_n = b_scale.stride(0);
  g.bs_stride_k = b_scale.stride(1);
  g.timeout_ns = (uint64_t)timeout_ns;
  g.error_flag = error_flag.data_ptr<int32_t>();
  cuda_check(b200::launch_fp8_gemm(g, at::cuda::getCurrentCUDAStream()), "fp8_gemm launch");
}

// ---------------------------------------------------------------------------------------
// CPU ranks over the shared-memory heap (host_ops.h)
// ---------------------------------------------------------------------------------------

b200::HostMoeLayout host_layout(const std::vector<int64_t>& offsets) {
  TORCH_CHECK(offsets.size() == 4, "expected offsets of (counts, expert_x, expert_meta, expert_y)");
  b200::HostMoeLayout lay;
  lay.counts = (uint64_t)offsets[0];
  lay.expert_x = (uint64_t)offsets[1];
  lay.expert_meta = (uint64_t)offsets[2];
  lay.expert_y = (uint64_t)offsets[3];
  return lay;
}

b200::HostMoeShape host_shape(const b200::HostShmHeap& heap, int64_t num_experts, int64_t topk, int64_t hidden,
                              int64_t max_recv, at::ScalarType in_dtype, at::ScalarType out_dtype) {
  TORCH_CHECK(num_experts > 0 && num_experts % heap.world_size() == 0, "num_experts must divide by the world size");
  TORCH_CHECK(topk > 0 && hidden > 0 && max_recv > 0, "bad MoE shape");
  b200::HostMoeShape s;
  s.num_experts = (int)num_experts;
  s.topk = (int)topk;
  s.hidden = (int)hidden;
  s.max_recv = (int)max_recv;
  s.in_dtype = dtype_code(in_dtype);
  s.out_dtype = dtype_code(out_dtype);
  return s;
}

void host_check_layout(const b200::HostShmHeap& heap, const b200::HostMoeLayout& lay, const b200::HostMoeShape& s) {
  const uint64_t El = (uint64_t)s.num_experts / heap.world_size();
  const uint64_t cells = El * (uint64_t)s.max_recv;
  const uint64_t end_counts = lay.counts + (uint64_t)heap.world_size() * s.num_experts * 4;
  const uint64_t end_x = lay.expert_x + cells * s.hidden * b200::host_dtype_bytes(s.in_dtype);
  const uint64_t end_meta = lay.expert_meta + cells * 5 * 4;
  const uint64_t end_y = lay.expert_y + cells * s.hidden * b200::host_dtype_bytes(s.out_dtype);
  TORCH_CHECK(lay.counts >= b200::kHeapHeaderBytes && end_counts <= heap.bytes() && end_x <= heap.bytes() &&
                  end_meta <= heap.bytes() && end_y <= heap.bytes(),
              "MoE regions do not fit the shared-memory slab");
}

py::tuple host_moe_dispatch(b200::HostShmHeap& heap, std::vector<int64_t> offsets, const at::Tensor& x,
                            const at::Tensor& indices, int64_t num_experts, int64_t max_recv,
                            at::ScalarType out_dtype, int64_t epoch, int64_t timeout_ns) {
  TORCH_CHECK(x.device().is_cpu() && indices.device().is_cpu(), "host_moe_dispatch takes CPU tensors");
  TORCH_CHECK(x.dim() == 2 && indices.dim() == 2 && x.is_contiguous(), "x [tokens, hidden] contiguous, indices [tokens, k]");
  TORCH_CHECK(indices.size(0) <= x.size(0), "more index rows than tokens");
  const b200::HostMoeLayout lay = host_layout(offsets);
  const b200::HostMoeShape s = host_shape(heap, num_experts, indices.size(1), x.size(1), max_recv, x.scalar_type(), out_dtype);
  host_check_layout(heap, lay, s);
  const at::Tensor idx = indices.to(at::kInt).contiguous();
  const int num_tokens = (int)idx.size(0);
  at::Tensor route = at::empty({(int64_t)num_tokens * s.topk, 3}, at::TensorOptions().dtype(at::kInt));
  at::Tensor expert_num = at::empty({s.num_experts / heap.world_size()}, at::TensorOptions().dtype(at::kInt));
  b200::StatusWord w;
  {
    py::gil_scoped_release release;
    w = b200::host_moe_dispatch(heap, lay, s, x.data_ptr(), idx.data_ptr<int32_t>(), num_tokens,
                                route.data_ptr<int32_t>(), expert_num.data_ptr<int32_t>(), (uint64_t)epoch,
                                (uint64_t)timeout_ns);
  }
  return py::make_tuple(status_to_dict(w), route, expert_num);
}

at::Tensor host_region(b200::HostShmHeap& heap, uint64_t offset, std::vector<int64_t> shape, at::ScalarType dtype) {
  return at::from_blob(heap.base(heap.rank()) + offset, shape, at::TensorOptions().dtype(dtype).device(at::kCPU));
}

void host_moe_expert_scale(b200::HostShmHeap& heap, std::vector<int64_t> offsets, int64_t num_experts, int64_t topk,
                           int64_t hidden, int64_t max_recv, at::ScalarType in_dtype, at::ScalarType out_dtype,
                           const at::Tensor& expert_num_tokens, double scale) {
  const b200::HostMoeLayout lay = host_layout(offsets);
  const b200::HostMoeShape s = host_shape(heap, num_experts, topk, hidden, max_recv, in_dtype, out_dtype);
  host_check_layout(heap, lay, s);
  const int64_t El = s.num_experts / heap.world_size();
  TORCH_CHECK(expert_num_tokens.scalar_type() == at::kInt && expert_num_tokens.is_contiguous() &&
                  expert_num_tokens.numel() == El,
              "expert_num_tokens must be int32 [local experts]");
  at::Tensor x = host_region(heap, lay.expert_x, {El, max_recv, hidden}, in_dtype);
  at::Tensor y = host_region(heap, lay.expert_y, {El, max_recv, hidden}, out_dtype);
  const int32_t* num = expert_num_tokens.data_ptr<int32_t>();
  if (El * max_recv * hidden <= (1 << 18)) {
    // small buffers: two calls over everything cost less than two per expert; rows past the
    // counts hold stale values that nobody reads
    y.copy_(x);
    y.mul_(scale);
    return;
  }
  for (int64_t el = 0; el < El; ++el) {
    const int64_t rows = std::min<int64_t>(std::max<int32_t>(num[el], 0), max_recv);
    if (rows == 0) continue;
    // the reference converts to the output type first and multiplies in that type
    // (all2all/reference.py:265)
    at::Tensor ys = y.select(0, el).narrow(0, 0, rows);
    ys.copy_(x.select(0, el).narrow(0, 0, rows));
    ys.mul_(scale);
  }
}

py::dict host_moe_combine(b200::HostShmHeap& heap, std::vector<int64_t> offsets, int64_t num_experts, int64_t max_recv,
                          at::ScalarType in_dtype, const at::Tensor& route, const at::Tensor& weights, at::Tensor out,
                          int64_t epoch, int64_t timeout_ns) {
  TORCH_CHECK(out.device().is_cpu() && out.dim() == 2 && out.is_contiguous(), "out [tokens, hidden] contiguous on CPU");
  TORCH_CHECK(weights.dim() == 2 && weights.scalar_type() == at::kFloat && weights.is_contiguous(),
              "weights must be float32 [tokens, k] contiguous");
  const int num_tokens = (int)weights.size(0);
  TORCH_CHECK(out.size(0) >= num_tokens, "out has fewer rows than weights");
  TORCH_CHECK(route.scalar_type() == at::kInt && route.is_contiguous() && route.dim() == 2 && route.size(1) == 3 &&
                  route.size(0) == (int64_t)num_tokens * weights.size(1),
              "route must be the int32 [tokens * k, 3] table returned by dispatch");
  const b200::HostMoeLayout lay = host_layout(offsets);
  const b200::HostMoeShape s = host_shape(heap, num_experts, weights.size(1), out.size(1), max_recv, in_dtype, out.scalar_type());
  host_check_layout(heap, lay, s);
  // a route table is only as good as its producer: owners, experts and slots must be in range
  {
    const int32_t* r = route.data_ptr<int32_t>();
    const int El = s.num_experts / heap.world_size();
    for (int64_t i = 0; i < route.size(0); ++i) {
      TORCH_CHECK(r[3 * i] < heap.world_size() && (r[3 * i] < 0 || (r[3 * i + 1] >= 0 && r[3 * i + 1] < El &&
                                                                   r[3 * i + 2] >= 0 && r[3 * i + 2] < s.max_recv)),
                  "route entry ", i, " is out of range");
    }
  }
  at::Tensor rows = at::empty({(int64_t)num_tokens, (int64_t)s.topk, (int64_t)s.hidden}, out.options());
  b200::StatusWord w;
  {
    py::gil_scoped_release release;
    w = b200::host_moe_pull(heap, lay, s, route.data_ptr<int32_t>(), num_tokens, rows.data_ptr(), (uint64_t)epoch,
                            (uint64_t)timeout_ns);
  }
  if (w.code == b200::STATUS_OK && num_tokens > 0) {
    // fp32 accumulator, k ascending, one rounding
    at::Tensor acc = at::zeros({(int64_t)num_tokens, (int64_t)s.hidden}, out.options().dtype(at::kFloat));
    for (int64_t j = 0; j < s.topk; ++j) {
      acc.addcmul_(rows.select(1, j).to(at::kFloat), weights.select(1, j).unsqueeze(1));
    }
    out.narrow(0, 0, num_tokens).copy_(acc);
  }
  return status_to_dict(w);
}

// ---- "dedup" protocol on CPU ranks ------------------------------------------------------

struct HostDedupGeometry {
  b200::HostMoeDedupLayout lay;
  b200::HostMoeDedupShape shape;
  int64_t ret_elem_bytes;
};

HostDedupGeometry host_dedup_geometry(const b200::HostShmHeap& heap, const std::vector<int64_t>& offsets, int64_t num_experts,
                                      int64_t topk, int64_t hidden, int64_t max_recv, int64_t max_tokens,
                                      at::ScalarType in_dtype, at::ScalarType out_dtype, bool partial_fp32, int64_t chunks) {
  TORCH_CHECK(offsets.size() == 7, "expected offsets of (counts, expert_x, expert_meta, expert_y, land, tok_rec, ret)");
  TORCH_CHECK(num_experts > 0 && num_experts % heap.world_size() == 0, "num_experts must divide by the world size");
  TORCH_CHECK(topk > 0 && topk <= 15 && hidden > 0 && max_recv > 0 && max_tokens > 0 && max_tokens < (1 << 24), "bad MoE shape");
  HostDedupGeometry g;
  g.lay.counts = (uint64_t)offsets[0];
  g.lay.expert_x = (uint64_t)offsets[1];
  g.lay.expert_meta = (uint64_t)offsets[2];
  g.lay.expert_y = (uint64_t)offsets[3];
  g.lay.land = (uint64_t)offsets[4];
  g.lay.tok_rec = (uint64_t)offsets[5];
  g.lay.ret = (uint64_t)offsets[6];
  g.shape.num_experts = (int)num_experts;
  g.shape.topk = (int)topk;
  g.shape.hidden = (int)hidden;
  g.shape.max_recv = (int)max_recv;
  g.shape.max_tokens = (int)max_tokens;
  g.shape.rec_ints = (int)((1 + 2 * topk + 3) / 4 * 4);
  g.shape.in_dtype = dtype_code(in_dtype);
  g.shape.out_dtype = dtype_code(out_dtype);
  g.shape.chunks = (int)std::max<int64_t>(1, std::min<int64_t>(chunks, 8));
  g.ret_elem_bytes = partial_fp32 ? 4 : b200::host_dtype_bytes(g.shape.out_dtype);
  const uint64_t ws = (uint64_t)heap.world_size();
  const uint64_t cells = (uint64_t)(num_experts / heap.world_size()) * (uint64_t)max_recv;
  const uint64_t toks = ws * (uint64_t)max_tokens;
  const uint64_t ends[7] = {
      g.lay.counts + ws * (uint64_t)num_experts * 4,
      g.lay.expert_x + cells * hidden * b200::host_dtype_bytes(g.shape.in_dtype),
      g.lay.expert_meta + cells * 5 * 4,
      g.lay.expert_y + cells * hidden * b200::host_dtype_bytes(g.shape.out_dtype),
      g.lay.land + toks * hidden * b200::host_dtype_bytes(g.shape.in_dtype),
      g.lay.tok_rec + toks * g.shape.rec_ints * 4,
      g.lay.ret + toks * hidden * (uint64_t)g.ret_elem_bytes,
  };
  TORCH_CHECK(g.lay.counts >= b200::kHeapHeaderBytes, "MoE regions overlap the slab header");
  for (uint64_t e : ends) TORCH_CHECK(e <= heap.bytes(), "MoE regions do not fit the shared-memory slab");
  return g;
}

py::tuple host_moe_dedup_dispatch(b200::HostShmHeap& heap, std::vector<int64_t> offsets, const at::Tensor& x,
                                  const at::Tensor& indices, int64_t num_experts, int64_t max_recv, int64_t max_tokens,
                                  at::ScalarType out_dtype, int64_t chunks, int64_t epoch, int64_t timeout_ns) {
  TORCH_CHECK(x.device().is_cpu() && indices.device().is_cpu(), "host_moe_dedup_dispatch takes CPU tensors");
  TORCH_CHECK(x.dim() == 2 && indices.dim() == 2 && x.is_contiguous(), "x [tokens, hidden] contiguous, indices [tokens, k]");
  TORCH_CHECK(indices.size(0) <= x.size(0) && indices.size(0) <= max_tokens, "more index rows than tokens / max_tokens");
  const HostDedupGeometry g = host_dedup_geometry(heap, offsets, num_experts, indices.size(1), x.size(1), max_recv, max_tokens,
                                                  x.scalar_type(), out_dtype, false, chunks);
  const at::Tensor idx = indices.to(at::kInt).contiguous();
  const int num_tokens = (int)idx.size(0);
  at::Tensor route = at::empty({(int64_t)num_tokens * g.shape.topk, 2}, at::TensorOptions().dtype(at::kInt));
  at::Tensor expert_num = at::empty({g.shape.num_experts / heap.world_size()}, at::TensorOptions().dtype(at::kInt));
  b200::StatusWord w;
  {
    py::gil_scoped_release release;
    w = b200::host_moe_dedup_dispatch(heap, g.lay, g.shape, x.data_ptr(), idx.data_ptr<int32_t>(), num_tokens,
                                      route.data_ptr<int32_t>(), expert_num.data_ptr<int32_t>(), (uint64_t)epoch,
                                      (uint64_t)timeout_ns);
  }
  return py::make_tuple(status_to_dict(w), route, expert_num);
}

// Combine of the dedup protocol.  `expert_y` is any tensor of the dispatch layout (the owner
// reduces its own expert outputs, so it need not live in the slab).  Owner side: per landed
// (source, token) the fp32 sum over its local entries, ascending k, of weight * expert_y[row],
// stored as ONE row into the source's return buffer.  Source side: the rows of the owners it
// used are added in ascending rank order in fp32 and rounded once.
py::dict host_moe_dedup_combine(b200::HostShmHeap& heap, std::vector<int64_t> offsets, int64_t num_experts, int64_t max_recv,
                                int64_t max_tokens, at::ScalarType in_dtype, bool partial_fp32, const at::Tensor& route,
                                const at::Tensor& weights, const at::Tensor& expert_y, at::Tensor out,
                                int64_t dispatch_epoch, int64_t epoch, int64_t timeout_ns) {
  TORCH_CHECK(out.device().is_cpu() && out.dim() == 2 && out.is_contiguous(), "out [tokens, hidden] contiguous on CPU");
  TORCH_CHECK(weights.dim() == 2 && weights.scalar_type() == at::kFloat && weights.is_contiguous(),
              "weights must be float32 [tokens, k] contiguous");
  const int64_t num_tokens = weights.size(0), k = weights.size(1), hidden = out.size(1);
  TORCH_CHECK(out.size(0) >= num_tokens && num_tokens <= max_tokens, "out has fewer rows than weights, or too many tokens");
  TORCH_CHECK(route.scalar_type() == at::kInt && route.is_contiguous() && route.dim() == 2 && route.size(1) == 2 &&
                  route.size(0) == num_tokens * k,
              "route must be the int32 [tokens * k, 2] table returned by dispatch");
  const HostDedupGeometry g = host_dedup_geometry(heap, offsets, num_experts, k, hidden, max_recv, max_tokens, in_dtype,
                                                  out.scalar_type(), partial_fp32, 1);
  const int ws = heap.world_size(), rank = heap.rank();
  const int64_t total_rows = (int64_t)(g.shape.num_experts / ws) * g.shape.max_recv;
  TORCH_CHECK(expert_y.device().is_cpu() && expert_y.is_contiguous() && expert_y.scalar_type() == out.scalar_type() &&
                  expert_y.numel() == total_rows * hidden,
              "expert_y does not have the dispatch layout / out_dtype");
  b200::StatusWord w;
  {
    py::gil_scoped_release release;
    w = b200::host_moe_dedup_send_weights(heap, g.lay, g.shape, route.data_ptr<int32_t>(), weights.data_ptr<float>(),
                                          (int)num_tokens, (uint64_t)epoch, (uint64_t)timeout_ns);
  }
  if (w.code != b200::STATUS_OK) return status_to_dict(w);

  // owner side: the records landed by the dispatch this combine belongs to
  const at::ScalarType ret_dtype = partial_fp32 ? at::kFloat : out.scalar_type();
  at::Tensor rec = host_region(heap, g.lay.tok_rec, {(int64_t)ws * max_tokens, (int64_t)g.shape.rec_ints}, at::kInt);
  const int32_t mark = (int32_t)(uint32_t)(uint64_t)dispatch_epoch;
  at::Tensor live = at::nonzero(rec.select(1, 0).eq((int64_t)mark)).squeeze(1);  // flat (source, token) cells
  bool bad_row = false;
  if (live.numel() > 0) {
    at::Tensor mine = rec.index_select(0, live);
    at::Tensor rows = mine.narrow(1, 1, k).to(at::kLong);
    at::Tensor wts = mine.narrow(1, 1 + k, k).contiguous().view(at::kFloat);
    bad_row = rows.ge(total_rows).any().item<bool>();
    at::Tensor valid = rows.ge(0).logical_and(rows.lt(total_rows));
    at::Tensor y2 = expert_y.view({total_rows, hidden});
    at::Tensor acc = at::zeros({live.size(0), hidden}, at::TensorOptions().dtype(at::kFloat));
    for (int64_t kk = 0; kk < k; ++kk) {
      at::Tensor r = rows.select(1, kk).clamp(0, total_rows - 1);
      at::Tensor wk = wts.select(1, kk) * valid.select(1, kk).to(at::kFloat);
      acc.addcmul_(y2.index_select(0, r).to(at::kFloat), wk.unsqueeze(1));
    }
    at::Tensor any_valid = valid.any(1);
    at::Tensor src_of = at::floor_divide(live, max_tokens);
    at::Tensor tok_of = live - src_of * max_tokens;
    at::Tensor partial = acc.to(ret_dtype);
    for (int s = 0; s < ws; ++s) {
      at::Tensor pick = at::nonzero(src_of.eq(s).logical_and(any_valid)).squeeze(1);
      if (pick.numel() == 0) continue;
      // row (this rank, token) of the SOURCE's return buffer
      at::Tensor dst = at::from_blob(heap.base(s) + g.lay.ret + (uint64_t)rank * max_tokens * hidden * g.ret_elem_bytes,
                                     {max_tokens, hidden}, at::TensorOptions().dtype(ret_dtype));
      dst.index_copy_(0, tok_of.index_select(0, pick), partial.index_select(0, pick));
    }
  }
  {
    py::gil_scoped_release release;
    w = b200::host_moe_dedup_return(heap, (uint64_t)epoch, (uint64_t)timeout_ns);
  }
  if (w.code != b200::STATUS_OK) return status_to_dict(w);

  // source side: add the owners' rows, ascending rank
  if (num_tokens > 0) {
    at::Tensor rt = route.view({num_tokens, k, 2});
    at::Tensor owner = rt.select(2, 0), row = rt.select(2, 1);
    at::Tensor ret = host_region(heap, g.lay.ret, {(int64_t)ws, max_tokens, hidden}, ret_dtype);
    at::Tensor acc = at::zeros({num_tokens, hidden}, at::TensorOptions().dtype(at::kFloat));
    for (int d = 0; d < ws; ++d) {
      at::Tensor used = at::nonzero(owner.eq(d).logical_and(row.ge(0)).any(1)).squeeze(1);
      if (used.numel() == 0) continue;
      acc.index_add_(0, used, ret.select(0, d).index_select(0, used).to(at::kFloat));
    }
    out.narrow(0, 0, num_tokens).copy_(acc);
  }
  if (bad_row) {
    w.code = b200::STATUS_BAD_INDEX;
    w.phase = b200::PHASE_MOE_RETURN;
    w.peer = -1;
    w.epoch = (uint64_t)epoch;
  }
  return status_to_dict(w);
}

py::tuple host_reduce_scatter(b200::HostShmHeap& heap, int64_t stage_offset, int64_t stage_bytes, const at::Tensor& partial,
                              const c10::optional<at::Tensor>& bias_once, int64_t epoch, int64_t timeout_ns) {
  TORCH_CHECK(partial.device().is_cpu() && partial.dim() == 2 && partial.is_contiguous(), "partial [M, N] contiguous on CPU");
  const int ws = heap.world_size();
  const int64_t m = partial.size(0), n = partial.size(1);
  TORCH_CHECK(m % ws == 0, "M must divide by the world size");
  const int dt = dtype_code(partial.scalar_type());
  const int64_t need = m * n * b200::host_dtype_bytes(dt);  // world * (M / world) * N elements
  TORCH_CHECK(need <= stage_bytes, "staging region of ", stage_bytes, " bytes is smaller than the ", need, " needed");
  TORCH_CHECK(stage_offset >= (int64_t)b200::kHeapHeaderBytes && (uint64_t)(stage_offset + stage_bytes) <= heap.bytes(),
              "staging region outside the slab");
  at::Tensor bias_f32;
  if (bias_once.has_value() && bias_once->defined()) {
    TORCH_CHECK(bias_once->numel() == n, "bias must have N elements");
    bias_f32 = bias_once->to(at::kFloat).contiguous();
  }
  b200::StatusWord w;
  {
    py::gil_scoped_release release;
    w = b200::host_rs_exchange(heap, (uint64_t)stage_offset, partial.data_ptr(), (int)m, (int)n,
                               b200::host_dtype_bytes(dt), (uint64_t)epoch, (uint64_t)timeout_ns);
  }
  const int64_t rows = m / ws;
  if (w.code != b200::STATUS_OK) return py::make_tuple(status_to_dict(w), at::empty({rows, n}, partial.options()));
  // fp32 sum in rank order, one rounding
  at::Tensor stage = host_region(heap, (uint64_t)stage_offset, {ws, rows, n}, partial.scalar_type());
  at::Tensor acc = at::zeros({rows, n}, partial.options().dtype(at::kFloat));
  for (int src = 0; src < ws; ++src) {
    acc.add_(src == heap.rank() ? partial.narrow(0, src * rows, rows) : stage.select(0, src));
  }
  if (bias_f32.defined()) acc.add_(bias_f32);
  return py::make_tuple(status_to_dict(w), acc.to(partial.scalar_type()));
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "B200 (sm_100a) kernels and symmetric-memory runtime";
  m.attr("MAX_WORLD_SIZE") = b200::kMaxWorldSize;
  m.attr("HEAP_HEADER_BYTES") = (int64_t)b200::kHeapHeaderBytes;
  m.attr("GEMM_RS_BLOCK_M") = b200::kGemmRsBlockM;
  m.attr("GEMM_RS_BLOCK_N") = b200::kGemmRsBlockN;

  py::class_<SymmHeap, std::shared_ptr<SymmHeap>>(m, "SymmHeap")
      .def(py::init([](int rank, int world_size, int64_t bytes, int device) {
             return std::make_shared<SymmHeap>(rank, world_size, (uint64_t)bytes, device);
           }),
           py::arg("rank"), py::arg("world_size"), py::arg("bytes"), py::arg("device"))
      .def("ipc_handle", [](const SymmHeap& h) { return py::bytes(h.ipc_handle()); })
      .def("open_peers",
           [](SymmHeap& h, const std::vector<py::bytes>& handles) {
             std::vector<std::string> hs;
             for (const auto& b : handles) hs.push_back(std::string(b));
             h.open_peers(hs);
           })
      .def("close", &SymmHeap::close)
      .def("close_peers", &SymmHeap::close_peers)
      .def_property_readonly("rank", &SymmHeap::rank)
      .def_property_readonly("world_size", &SymmHeap::world_size)
      .def_property_readonly("device", &SymmHeap::device)
      .def_property_readonly("bytes", [](const SymmHeap& h) { return (int64_t)h.bytes(); })
      .def_property_readonly("peers_open", &SymmHeap::peers_open)
      .def("peer_base", [](const SymmHeap& h, int r) { return (int64_t)h.peer_base(r); })
      .def("view", &heap_view, py::arg("offset"), py::arg("shape"), py::arg("dtype"))
      .def("status", [](const SymmHeap& h) { return status_to_dict(h.status_host()); })
      .def("status_code", [](const SymmHeap& h) { return (int)h.status_host().code; })
      .def("status_sync", [](const SymmHeap& h) { return status_to_dict(h.status_sync()); })
      .def("reset_status", &SymmHeap::reset_status)
      .def("barrier",
           [](SymmHeap& h, int64_t epoch, int64_t timeout_ns) {
             c10::cuda::CUDAGuard guard(h.device());
             cuda_check(b200::launch_symm_barrier(h, (uint64_t)epoch, (uint64_t)timeout_ns,
                                                  at::cuda::getCurrentCUDAStream()),
                        "barrier launch");
           })
      .def("link_probe",
           [](SymmHeap& h, int peer, int64_t src_offset, int64_t dst_offset, int64_t bytes, int mode, int chunk, int grid,
              int64_t timeout_ns) {
             c10::cuda::CUDAGuard guard(h.device());
             cuda_check(b200::launch_link_probe(h, peer, (uint64_t)src_offset, (uint64_t)dst_offset, (uint64_t)bytes, mode,
                                                chunk, grid, (uint64_t)timeout_ns, at::cuda::getCurrentCUDAStream()),
                        "link_probe launch");
           })
      .def("wait_selftest", [](SymmHeap& h, int slot, int64_t want, int64_t timeout_ns) {
        c10::cuda::CUDAGuard guard(h.device());
        cuda_check(b200::launch_wait_selftest(h, slot, (uint64_t)want, (uint64_t)timeout_ns,
                                              at::cuda::getCurrentCUDAStream()),
                   "wait_selftest launch");
      });

  py::class_<b200::HostShmHeap, std::shared_ptr<b200::HostShmHeap>>(m, "HostShmHeap")
      .def(py::init([](const std::string& prefix, int rank, int world_size, int64_t bytes) {
             return std::make_shared<b200::HostShmHeap>(prefix, rank, world_size, (uint64_t)bytes);
           }),
           py::arg("prefix"), py::arg("rank"), py::arg("world_size"), py::arg("bytes"))
      .def("open_peers", [](b200::HostShmHeap& h, int64_t timeout_ns) { return h.open_peers((uint64_t)timeout_ns); })
      .def("close", &b200::HostShmHeap::close)
      .def("unlink", &b200::HostShmHeap::unlink)
      .def("signal", [](b200::HostShmHeap& h, int row, int dst, int64_t epoch) { h.signal(row, dst, (uint64_t)epoch); })
      .def("wait",
           [](b200::HostShmHeap& h, int row, int src, int64_t epoch, int64_t timeout_ns, int phase) {
             py::gil_scoped_release release;
             b200::StatusWord w = h.wait(row, src, (uint64_t)epoch, (uint64_t)timeout_ns, (uint32_t)phase);
             py::gil_scoped_acquire acquire;
             return status_to_dict(w);
           },
           py::arg("row"), py::arg("src"), py::arg("epoch"), py::arg("timeout_ns"), py::arg("phase") = (int)b200::PHASE_TEST)
      .def("barrier",
           [](b200::HostShmHeap& h, int64_t epoch, int64_t timeout_ns) {
             py::gil_scoped_release release;
             b200::StatusWord w = h.barrier((uint64_t)epoch, (uint64_t)timeout_ns);
             py::gil_scoped_acquire acquire;
             return status_to_dict(w);
           })
      .def("status", [](const b200::HostShmHeap& h) { return status_to_dict(h.last_status()); })
      .def("reset_status", &b200::HostShmHeap::reset_status)
      .def("view",
           [](b200::HostShmHeap& h, int r, int64_t offset, std::vector<int64_t> shape, at::ScalarType dtype) {
             int64_t numel = 1;
             for (auto s : shape) numel *= s;
             const int64_t nbytes = numel * (int64_t)c10::elementSize(dtype);
             TORCH_CHECK(r >= 0 && r < h.world_size() && h.base(r) != nullptr, "rank ", r, " is not mapped");
             TORCH_CHECK(offset >= (int64_t)b200::kHeapHeaderBytes && (uint64_t)(offset + nbytes) <= h.bytes(),
                         "view outside the payload area of the slab");
             return at::from_blob(h.base(r) + offset, shape, at::TensorOptions().dtype(dtype).device(at::kCPU));
           },
           py::arg("rank"), py::arg("offset"), py::arg("shape"), py::arg("dtype"));

  py::class_<MoeDedupEngine, std::shared_ptr<MoeDedupEngine>>(m, "MoeDedupEngine")
      .def(py::init<std::shared_ptr<SymmHeap>, int64_t, int64_t, int64_t, int64_t, int64_t, at::ScalarType, bool,
                    std::vector<int64_t>, at::Tensor, at::Tensor, at::Tensor, at::Tensor, int64_t>(),
           py::arg("heap"), py::arg("num_experts"), py::arg("topk"), py::arg("hidden"), py::arg("max_tokens"),
           py::arg("max_recv"), py::arg("dtype"), py::arg("partial_fp32"), py::arg("offsets"), py::arg("expert_y"),
           py::arg("blk_hist"), py::arg("route"), py::arg("expert_num_tokens"), py::arg("timeout_ns"))
      .def("dispatch", &MoeDedupEngine::dispatch, py::arg("x"), py::arg("indices"), py::arg("weights") = py::none(),
           py::arg("fuse_scale") = false, py::arg("scale") = 1.0)
      .def("combine", &MoeDedupEngine::combine, py::arg("out"), py::arg("weights"), py::arg("expert_y") = py::none())
      .def("forward", &MoeDedupEngine::forward)
      .def("set_trace", &MoeDedupEngine::set_trace, py::arg("dispatch_trace") = py::none(), py::arg("combine_trace") = py::none())
      .def("set_timeout_ns", &MoeDedupEngine::set_timeout_ns)
      .def_readwrite("bulk_landing", &MoeDedupEngine::bulk_landing)
      .def_readwrite("chunks", &MoeDedupEngine::chunks)
      .def_readwrite("chunk_min_ranks", &MoeDedupEngine::chunk_min_ranks)
      .def_readwrite("chunk_min_bytes", &MoeDedupEngine::chunk_min_bytes)
      .def_property_readonly("dispatch_epoch", &MoeDedupEngine::dispatch_epoch)
      .def_property_readonly("combine_epoch", &MoeDedupEngine::combine_epoch);
  m.def("moe_dedup_dispatch_max_blocks", [](int device, int num_experts, int num_entries, int bulk_landing) {
    c10::cuda::CUDAGuard guard(device);
    return b200::moe_dedup_dispatch_max_blocks(device, num_experts, num_entries, bulk_landing);
  });

  py::class_<GemmRsEngine, std::shared_ptr<GemmRsEngine>>(m, "GemmRsEngine")
      .def(py::init<std::shared_ptr<SymmHeap>, std::vector<int64_t>, std::vector<int64_t>, int64_t, int64_t, int64_t>(),
           py::arg("heap"), py::arg("stage_offsets"), py::arg("counter_offsets"), py::arg("stage_bytes"),
           py::arg("counter_bytes"), py::arg("timeout_ns"))
      .def("run", &GemmRsEngine::run, py::arg("a"), py::arg("w"), py::arg("bias"), py::arg("out"),
           py::arg("bias_at_source") = true, py::arg("bias_scale") = 1.0)
      .def("plan", &GemmRsEngine::plan)
      .def("set_trace", &GemmRsEngine::set_trace)
      .def("restart_epochs", &GemmRsEngine::restart_epochs)
      .def("set_mcast", &GemmRsEngine::set_mcast)
      .def_property_readonly("nvls", &GemmRsEngine::nvls)
      .def_property_readonly("epoch", &GemmRsEngine::epoch)
      .def_readwrite("max_ctas", &GemmRsEngine::max_ctas)
      .def_readwrite("block_n", &GemmRsEngine::block_n)
      .def_readwrite("cta_pair", &GemmRsEngine::cta_pair)
      .def_readwrite("splits", &GemmRsEngine::splits)
      .def_readwrite("debug", &GemmRsEngine::debug)
      .def_readwrite("fuse_own", &GemmRsEngine::fuse_own)
      .def_readwrite("tma_store", &GemmRsEngine::tma_store)
      .def_readwrite("force_staged", &GemmRsEngine::force_staged)
      .def_readwrite("checked", &GemmRsEngine::checked);

  py::class_<b200::McastRegion, std::shared_ptr<b200::McastRegion>>(m, "McastRegion")
      .def(py::init([](int rank, int world_size, int64_t bytes, int device) {
             return std::make_shared<b200::McastRegion>(rank, world_size, (uint64_t)bytes, device);
           }),
           py::arg("rank"), py::arg("world_size"), py::arg("bytes"), py::arg("device"))
      .def_static("supported",
                  [](int device) {
                    std::string why;
                    const bool ok = b200::McastRegion::supported(device, &why);
                    return py::make_tuple(ok, why);
                  })
      .def("create_and_export", &b200::McastRegion::create_and_export)
      .def("import_from", &b200::McastRegion::import_from)
      .def("add_device", &b200::McastRegion::add_device)
      .def("bind_and_map", &b200::McastRegion::bind_and_map)
      .def("close", &b200::McastRegion::close)
      .def_property_readonly("bytes", [](const b200::McastRegion& r) { return (int64_t)r.bytes(); })
      .def_property_readonly("mapped", &b200::McastRegion::mapped)
      .def_property_readonly("local_ptr", [](const b200::McastRegion& r) { return (int64_t)reinterpret_cast<uintptr_t>(r.local_ptr()); })
      .def_property_readonly("mc_ptr", [](const b200::McastRegion& r) { return (int64_t)reinterpret_cast<uintptr_t>(r.mc_ptr()); })
      .def("view",
           [](b200::McastRegion& r, int64_t offset, std::vector<int64_t> shape, at::ScalarType dtype) {
             int64_t numel = 1;
             for (auto s : shape) numel *= s;
             const int64_t nbytes = numel * (int64_t)c10::elementSize(dtype);
             TORCH_CHECK(r.mapped() && offset >= 0 && (uint64_t)(offset + nbytes) <= r.bytes(), "view outside the region");
             auto opts = at::TensorOptions().dtype(dtype).device(at::kCUDA, r.device());
             return at::from_blob(static_cast<uint8_t*>(r.local_ptr()) + offset, shape, opts);
           },
           py::arg("offset"), py::arg("shape"), py::arg("dtype"))
      .def("reduce_selftest", [](b200::McastRegion& r, int64_t offset, at::Tensor out) {
        TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.scalar_type() == at::kBFloat16 && out.numel() % 8 == 0,
                    "out must be a contiguous bf16 CUDA tensor with a multiple of 8 elements");
        c10::cuda::CUDAGuard guard(r.device());
        cuda_check(b200::launch_mcast_selftest(r, (uint64_t)offset, out.data_ptr(), (uint64_t)(out.numel() / 8),
                                               at::cuda::getCurrentCUDAStream()),
                   "mcast selftest launch");
      });

  m.attr("FLAG_BARRIER") = (int)b200::FLAG_BARRIER;
  m.attr("FLAG_TEST") = (int)b200::FLAG_TEST;
  m.def("host_moe_dispatch", &host_moe_dispatch);
  m.def("host_moe_expert_scale", &host_moe_expert_scale);
  m.def("host_moe_combine", &host_moe_combine);
  m.def("host_moe_dedup_dispatch", &host_moe_dedup_dispatch);
  m.def("host_moe_dedup_combine", &host_moe_dedup_combine);
  m.def("host_reduce_scatter", &host_reduce_scatter);
  m.def("moe_dispatch", &moe_dispatch);
  m.def("moe_expert_scale", &moe_expert_scale);
  m.def("moe_combine", &moe_combine);
  m.def("moe_forward", &moe_forward);
  m.def("gemm_rs", &gemm_rs);
  m.def("fp8_gemm", &fp8_gemm);
  m.def("gemm_rs_plan", [](int64_t M, int64_t N, int64_t K, int64_t ws, int64_t block_n, int64_t cta_pair, int64_t splits) {
    const b200::GemmRsPlan p = b200::gemm_rs_plan((int)M, (int)N, (int)K, (int)ws, (int)block_n, (int)cta_pair, (int)splits);
    py::dict d;
    d["block_n"] = p.block_n;
    d["cta_pair"] = p.cta_pair;
    d["splits"] = p.splits;
    d["stage_bytes"] = (int64_t)p.stage_bytes;
    d["counter_bytes"] = (int64_t)p.counter_bytes;
    return d;
  });
}
