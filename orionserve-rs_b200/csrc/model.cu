// Device model: weights, paged KV arena, RoPE tables, work buffers and the
// per-step kernel sequence. Mirrors TransformerModel::{new, forward}
// (crates/orion-models/src/transformer.rs:148-177, 230-442) with every tensor
// operation on the GPU; the host only validates the batch, resolves slots
// (attention.rs:182-186) and launches.
#include "model.h"

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <tuple>

namespace orion {

int compute_layout(uint32_t heads, uint32_t kv_heads, uint32_t ffn, uint32_t rank, uint32_t world,
                   ParallelLayout *out) {
  // Rank::new (orion-distributed/src/lib.rs:74-90)
  if (world == 0) return set_error(ORION_ERR_INVALID_REQUEST, "world_size must be at least 1");
  if (rank >= world)
    return set_error(ORION_ERR_INVALID_REQUEST, "rank %u is out of range for world size %u", rank,
                     world);
  if (world == 1) {  // lib.rs:175-190
    *out = ParallelLayout{{0, heads}, {0, kv_heads}, {0, ffn}};
    return ORION_OK;
  }
  if (kv_heads < world)  // lib.rs:193-200
    return set_error(ORION_ERR_INVALID_REQUEST,
                     "model has %u KV heads but world size is %u; tensor parallelism beyond the KV "
                     "head count would require replicating them, which is not implemented",
                     kv_heads, world);
  auto shard = [&](uint32_t total, Shard *s) -> int {  // shard_dimension, lib.rs:139-152
    if (total % world != 0)
      return set_error(ORION_ERR_INVALID_REQUEST,
                       "cannot split %u evenly across %u ranks; tensor parallelism requires the "
                       "dimension to be divisible by the world size",
                       total, world);
    s->len = total / world;
    s->start = (uint64_t)rank * s->len;
    return ORION_OK;
  };
  ORION_TRY(shard(heads, &out->query_heads));
  ORION_TRY(shard(kv_heads, &out->kv_heads));
  ORION_TRY(shard(ffn, &out->ffn));
  return ORION_OK;
}

// Tuning A/B: ORION_FUSE_QKV=0 keeps the separate RoPE / KV-write kernel before decode attention.
bool g_fuse_qkv = std::getenv("ORION_FUSE_QKV") ? std::atoi(std::getenv("ORION_FUSE_QKV")) != 0 : true;
// Tuning A/B: ORION_FUSE_SWIGLU=0 keeps the separate SwiGLU kernel after the gate/up projection.
bool g_fuse_swiglu = std::getenv("ORION_FUSE_SWIGLU") ? std::atoi(std::getenv("ORION_FUSE_SWIGLU")) != 0 : true;
// Tuning A/B: ORION_STEP_GRAPH=0 launches every decode step kernel by kernel.
bool g_step_graph = std::getenv("ORION_STEP_GRAPH") ? std::atoi(std::getenv("ORION_STEP_GRAPH")) != 0 : true;
// Capture and instantiation take about 12 ms and save 0.09 ms per step: only a layout that stays is worth it.
// ORION_STEP_GRAPH_AFTER overrides the number of repeats (the parity tests use 2).
const uint32_t kGraphAfterSteps = std::getenv("ORION_STEP_GRAPH_AFTER") ? (uint32_t)std::max(1, std::atoi(std::getenv("ORION_STEP_GRAPH_AFTER"))) : 32u;
constexpr size_t kMaxStepGraphs = 16;
// Tuning A/B: ORION_READY_COUNTERS=0 makes the projection after a tensor-parallel hand-over wait for that
// kernel's completion again instead of polling its count of finished rows.
bool g_ready_counters = std::getenv("ORION_READY_COUNTERS") ? std::atoi(std::getenv("ORION_READY_COUNTERS")) != 0 : true;

namespace {

template <typename T>
struct DTypeOf;
template <>
struct DTypeOf<float> { static constexpr int value = ORION_DTYPE_F32; static constexpr bool is_bf16 = false; };
template <>
struct DTypeOf<bf16> { static constexpr int value = ORION_DTYPE_BF16; static constexpr bool is_bf16 = true; };

size_t dtype_size(int dtype) {
  switch (dtype) {
    case ORION_DTYPE_F32: return 4;
    case ORION_DTYPE_F16:
    case ORION_DTYPE_BF16: return 2;
    default: return 0;
  }
}

enum : uint32_t {
  kGotInNorm = 1u << 0, kGotPostNorm = 1u << 1, kGotQ = 1u << 2, kGotK = 1u << 3, kGotV = 1u << 4,
  kGotO = 1u << 5, kGotGate = 1u << 6, kGotUp = 1u << 7, kGotDown = 1u << 8,
  kGotAllLayer = (1u << 9) - 1,
};

template <typename T>
class Model final : public ModelBase {
 public:
  // Only the ordinal is kept: the model may outlive the backend handle it was created from.
  Model(OrionBackend *backend, const OrionModelDesc &d) : ordinal_(backend->ordinal), d_(d) {}
  ~Model() override {
    cudaSetDevice(ordinal_);
    if (stream_) cudaStreamSynchronize(stream_);
    drop_graphs();
    for (void *p : ipc_opened_) cudaIpcCloseMemHandle(p);
    for (void *p : allocs_) cudaFree(p);
    if (h_meta_) cudaFreeHost(h_meta_);
    if (stage_raw_) cudaFree(stage_raw_);
    if (stage_f32_) cudaFree(stage_f32_);
    for (cudaEvent_t e : head_ev_)
      if (e) cudaEventDestroy(e);
    if (copy_stream_) cudaStreamDestroy(copy_stream_);
    if (ev0_) cudaEventDestroy(ev0_);
    if (ev1_) cudaEventDestroy(ev1_);
    for (cudaEvent_t e : prof_pool_) cudaEventDestroy(e);
    if (stream_) cudaStreamDestroy(stream_);
  }

  int init();
  int load_tensor(const char *name, int dtype, const uint64_t *shape, int ndim,
                  const void *data) override;
  int init_random(uint64_t seed, float std) override;
  int finalize() override;
  int forward(const BatchView &b, float *logits_out, uint64_t logits_capacity,
              uint32_t *token_ids_out) override;
  int replay(int iterations, uint32_t category_mask, float *elapsed_ms) override;
  int profile(int iterations, float category_ms[kProfCategories],
              uint64_t category_launches[kProfCategories]) override;
  int fill_kv_random(uint64_t seed, float std) override;
  int read_kv(float *out, uint64_t capacity) override;
  uint64_t last_launch_count() const override { return last_launches_; }
  const OrionModelDesc &desc() const override { return d_; }

 private:
  // bf16 build: gate and up rows alternate in w_gu so that the GEMM epilogue can apply SwiGLU.
  static constexpr bool kInterleaveGateUp = sizeof(T) == 2;
  T *gu_stage_ = nullptr;  // upload staging for one gate or up matrix
  struct Layer {
    T *w_qkv = nullptr, *w_o = nullptr, *w_gu = nullptr, *w_down = nullptr;
    float *b_qkv = nullptr, *in_norm = nullptr, *post_norm = nullptr;
    uint32_t got = 0;
    bool any_bias = false;
  };

  template <typename U>
  int alloc(U **p, size_t count) {
    void *raw = nullptr;
    ORION_CUDA_CHECK("allocate", cudaMalloc(&raw, (count ? count : 1) * sizeof(U)));
    allocs_.push_back(raw);
    *p = static_cast<U *>(raw);
    return ORION_OK;
  }
  int ensure_stage(void **buf, size_t *cap, size_t bytes) {
    if (*cap >= bytes) return ORION_OK;
    if (*buf) cudaFree(*buf);
    *buf = nullptr;
    *cap = 0;
    ORION_CUDA_CHECK("allocate staging", cudaMalloc(buf, bytes));
    *cap = bytes;
    return ORION_OK;
  }
  // Copies rows [r0,r1) x cols [c0,c1) of a host [R][C] tensor of `dtype` into a
  // contiguous device destination (`dst_t` of T or `dst_f`, whichever is non-null),
  // converting once at load like the reference's loader (loader.rs:74-96).
  int upload_slice(T *dst_t, float *dst_f, const void *src, int dtype, uint64_t C, uint64_t r0,
                   uint64_t r1, uint64_t c0, uint64_t c1);
  // part 0: the whole step; 1: the embedding and the layers (what a step graph holds); 2: the LM head and what follows
  int run_step_body(bool want_argmax, int part = 0);
  int run_step_graphed(bool want_argmax);
  int run_step(bool want_argmax) {
    const int rc = graph_eligible() ? run_step_graphed(want_argmax) : run_step_body(want_argmax);
    // a fused hand-over sequence that stopped half way leaves the device-resident epoch behind the inboxes: the ranks
    // cannot be brought back in step from here
    if (rc != ORION_OK && nccl_ && tp_fused_) tp_broken_ = true;
    return rc;
  }
  // Pure decode steps on one GPU replay a CUDA graph of the embedding and the layers once the same batch layout has
  // come 32 times in a row: every kernel argument of such a step is a pointer into buffers that do not move (the
  // step's tokens, positions and block tables are uploaded into the metadata array before the launch), so the graph
  // holds for as long as the layout (rows, sequences, offsets inside the metadata array, context splits) does.
  struct GraphKey {
    uint32_t rows, seqs, splits, blocks_per_split, generation;
    size_t offsets[8];  // [7] is the address of the metadata array, the others are offsets inside it
    bool operator<(const GraphKey &o) const {
      return std::tie(rows, seqs, splits, blocks_per_split, generation, offsets[0], offsets[1], offsets[2], offsets[3], offsets[4],
                      offsets[5], offsets[6], offsets[7]) <
             std::tie(o.rows, o.seqs, o.splits, o.blocks_per_split, o.generation, o.offsets[0], o.offsets[1], o.offsets[2], o.offsets[3],
                      o.offsets[4], o.offsets[5], o.offsets[6], o.offsets[7]);
    }
    bool operator==(const GraphKey &o) const { return !(*this < o) && !(o < *this); }
  };
  struct StepGraph {
    cudaGraphExec_t exec = nullptr;
    uint64_t launches = 0;
  };
  std::map<GraphKey, StepGraph> graphs_;
  GraphKey last_key_{};
  uint32_t key_streak_ = 0;
  bool graph_eligible() const {
    // under tensor parallelism only steps that hand over through peer memory (no NCCL call inside the step)
    return g_step_graph && DTypeOf<T>::is_bf16 && meta_.decode && !meta_.zero_count && !prof_on_ && only_mask_ == 0 &&
           (!nccl_ || (tp_fused_ && meta_.rows <= kTpFusedMaxRows)) && decode_attention_supported(kv_, lq_);
  }
  void step_decode_plan(uint32_t *splits, uint32_t *blocks_per_split) const {
    const DecodePlan dp = decode_plan(meta_.rows, lkv_, meta_.total_blocks, meta_.max_position, d_.block_size, 32);
    uint32_t want = dp.splits;
    while (want > 1 && decode_scratch_floats(meta_.rows, lq_, d_.head_dim, want) > dscratch_floats_) --want;
    *splits = want;
    *blocks_per_split = dp.blocks_per_split;
  }
  GraphKey layout_key() const {
    GraphKey key{};
    key.rows = meta_.rows, key.seqs = meta_.seqs, key.generation = g_tuning_generation;
    step_decode_plan(&key.splits, &key.blocks_per_split);
    // meta_.tables follows meta_.offsets at a distance that only depends on the sequence count, so it needs no slot
    const size_t offs[8] = {meta_.tokens, meta_.positions, meta_.slot_block, meta_.slot_slot, meta_.seq_of_row, meta_.last_rows,
                            meta_.offsets, reinterpret_cast<size_t>(d_meta_)};
    for (int i = 0; i < 8; ++i) key.offsets[i] = offs[i];
    return key;
  }
  void drop_graphs() {
    for (auto &g : graphs_)
      if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
    graphs_.clear();
  }
  // Waits for a stream of this model. Under tensor parallelism the wait watches the communicator
  // and is bounded in time, so a peer that died cannot hold the host inside a blocking synchronise.
  int wait_for(cudaStream_t s, const char *stage) {
    if (nccl_) return nccl_->wait_stream(s, stage);
    ORION_CUDA_CHECK(stage, cudaStreamSynchronize(s));
    return ORION_OK;
  }
  int tp_reduce(uint32_t *splits, size_t slab);
  int setup_peer_handover();
  // Row-parallel projection -> residual + norm. Single GPU: the fused residual/norm kernel.
  // Tensor parallel: the fused peer-memory all-reduce + residual + norm kernel, or NCCL followed
  // by the single-GPU kernel. `out_rows`/`row_map` select gathered output rows (final norm).
  int handover(uint32_t splits, const float *norm_w, T *out, const uint32_t *row_map, uint32_t out_rows, bool count_ready = false);
  // The running total of finished hand-over CTAs the next projection has to see (ReadyWait in common.cuh).
  uint32_t *ready_ = nullptr;
  // Device state of the fused hand-overs: [0] the epoch of the step's first hand-over, [1] the count of finished
  // hand-over rows at the start of the step; advanced on the device at the end of every step (launch_tp_state_bump), so
  // that a step's launches take the same arguments every time. The host only counts within a step.
  uint32_t *tp_state_ = nullptr;
  uint32_t step_epochs_ = 0, step_rows_counted_ = 0;
  bool tp_broken_ = false;
  // Vocabulary-parallel LM head under tensor parallelism: this rank holds rows [head_v0_, head_v0_ + head_vn_)
  // of the head, computes that column block of the logits and stores it straight into the leader's
  // logits buffer (peer-mapped); flags in the leader's memory tell it when every block has landed.
  bool head_parallel_ = false;
  uint32_t head_v0_ = 0, head_vn_ = 0;
  float *head_out_ = nullptr;       // the leader's logits buffer as seen from this rank
  uint32_t *head_flags_ = nullptr;  // the leader's flag words as seen from this rank (own allocation on the leader)
  uint32_t head_epoch_ = 1;
  int setup_head_peers();
  TpPeers peers_{};
  uint32_t *tp_inbox_ = nullptr;  // where the peers push their partial sums (peer-mapped)
  bool tp_fused_ = false;
  bool tp_two_shot_ = false;
  std::vector<void *> ipc_opened_;
  // Per-launch event pairs of a profiled step, resolved after the stream drains.
  struct ProfRec { int cat; cudaEvent_t a, b; };
  std::vector<ProfRec> prof_recs_;
  std::vector<cudaEvent_t> prof_pool_;
  size_t prof_used_ = 0;
  bool prof_on_ = false;
  uint32_t only_mask_ = 0;  // non-zero: launch only these kernel categories (timing replays)
  cudaEvent_t prof_event() {
    if (prof_used_ == prof_pool_.size()) {
      cudaEvent_t e = nullptr;
      cudaEventCreate(&e);
      prof_pool_.push_back(e);
    }
    return prof_pool_[prof_used_++];
  }
  template <typename F>
  int timed(int cat, F &&fn) {
    // Timing only: a replay restricted to some kernel categories launches just those, back to
    // back, on whatever the buffers hold (the results are meaningless, the shapes are the step's).
    if (only_mask_ && !(only_mask_ & (1u << cat))) return ORION_OK;
    if (!prof_on_) return fn();
    cudaEvent_t a = prof_event(), b = prof_event();
    cudaEventRecord(a, stream_);
    const int rc = fn();
    cudaEventRecord(b, stream_);
    prof_recs_.push_back({cat, a, b});
    return rc;
  }

  int ordinal_;
  OrionModelDesc d_;
  cudaStream_t stream_ = nullptr;
  // LM head in column blocks with the download of block i overlapping the computation of i + 1
  static constexpr int kHeadChunks = 4;
  cudaStream_t copy_stream_ = nullptr;
  cudaEvent_t head_ev_[kHeadChunks] = {};
  uint32_t head_off_[kHeadChunks] = {}, head_cols_[kHeadChunks] = {};
  int head_chunks_ = 0;
  cudaEvent_t ev0_ = nullptr, ev1_ = nullptr;
  std::vector<void *> allocs_;
  ParallelLayout lay_;
  uint32_t lq_ = 0, lkv_ = 0, lf_ = 0;
  KvLayout kv_{};

  std::vector<Layer> layers_;
  T *embed_ = nullptr, *lm_head_ = nullptr, *lm_head_own_ = nullptr;
  float *final_norm_ = nullptr;
  bool got_embed_ = false, got_head_ = false, got_final_norm_ = false, finalized_ = false;
  T *arena_ = nullptr;
  float *rope_cos_ = nullptr, *rope_sin_ = nullptr;

  // work buffers
  float *hidden_ = nullptr, *partial_ = nullptr, *logits_ = nullptr, *dscratch_ = nullptr;
  T *normed_ = nullptr, *qbuf_ = nullptr, *attn_ = nullptr, *act_ = nullptr, *tail_ = nullptr;
  uint32_t *argmax_ = nullptr;
  size_t partial_floats_ = 0, dscratch_floats_ = 0;

  // batch metadata: one u32 array on the device, filled from a pinned mirror
  uint32_t *d_meta_ = nullptr, *h_meta_ = nullptr;
  size_t meta_cap_ = 0;
  struct Meta {
    uint32_t rows = 0, seqs = 0, max_position = 0;
    uint64_t total_blocks = 0;  // sum over the rows of the blocks their contexts span
    bool decode = false, zero_count = false;
    size_t tokens = 0, positions = 0, slot_block = 0, slot_slot = 0, seq_of_row = 0, last_rows = 0,
           offsets = 0, tables = 0, tiles = 0, total = 0;
    uint32_t num_tiles = 0;  // prefill attention tiles (0 = the batch does not use that kernel)
    // Mixed batches: a run of one-token sequences at the head or the tail of the batch (the
    // scheduler puts all decodes before or after all prefills, scheduler.rs:244-250) goes to
    // the decode attention kernel, the other rows to the prefill kernel.
    uint32_t dec_row0 = 0, dec_rows = 0;
  } meta_;

  void *stage_raw_ = nullptr, *stage_f32_ = nullptr;
  size_t stage_raw_cap_ = 0, stage_f32_cap_ = 0;
  std::unique_ptr<NcclCollective> nccl_;
  uint64_t last_launches_ = 0;
};

template <typename T>
int Model<T>::init() {
  const OrionModelDesc &d = d_;
  if (d.hidden_size == 0 || d.num_layers == 0 || d.num_attention_heads == 0 ||
      d.num_kv_heads == 0 || d.head_dim == 0 || d.vocab_size == 0 || d.ffn_dim == 0)
    return set_error(ORION_ERR_MODEL, "config.json is malformed: a model dimension is zero");
  if (d.num_attention_heads % d.num_kv_heads != 0)  // config.rs:203-208
    return set_error(ORION_ERR_MODEL,
                     "config.json is malformed: num_attention_heads (%u) must be a multiple of "
                     "num_key_value_heads (%u)",
                     d.num_attention_heads, d.num_kv_heads);
  if (d.head_dim % 2 != 0)  // tensor.rs:229-233
    return set_error(ORION_ERR_MODEL, "config.json is malformed: RoPE requires an even head_dim, got %u",
                     d.head_dim);
  if (d.block_size == 0 || d.max_batch_tokens == 0 || d.max_batch_sequences == 0)
    return set_error(ORION_ERR_INVALID_REQUEST,
                     "block_size, max_batch_tokens and max_batch_sequences must be non-zero");
  ORION_TRY(compute_layout(d.num_attention_heads, d.num_kv_heads, d.ffn_dim, d.tp_rank, d.tp_world,
                           &lay_));
  lq_ = (uint32_t)lay_.query_heads.len;
  lkv_ = (uint32_t)lay_.kv_heads.len;
  lf_ = (uint32_t)lay_.ffn.len;

  ORION_CUDA_CHECK("set device", cudaSetDevice(ordinal_));
  ORION_CUDA_CHECK("create stream", cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
  ORION_CUDA_CHECK("create stream", cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking));
  for (cudaEvent_t &e : head_ev_) ORION_CUDA_CHECK("create event", cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  ORION_CUDA_CHECK("create event", cudaEventCreate(&ev0_));
  ORION_CUDA_CHECK("create event", cudaEventCreate(&ev1_));

  const size_t H = d.hidden_size, hd = d.head_dim, V = d.vocab_size;
  const size_t nqkv = (size_t)(lq_ + 2 * lkv_) * hd;
  layers_.resize(d.num_layers);
  for (Layer &L : layers_) {
    ORION_TRY(alloc(&L.w_qkv, nqkv * H));
    ORION_TRY(alloc(&L.w_o, H * lq_ * hd));
    ORION_TRY(alloc(&L.w_gu, (size_t)2 * lf_ * H));
    ORION_TRY(alloc(&L.w_down, H * lf_));
    ORION_TRY(alloc(&L.in_norm, H));
    ORION_TRY(alloc(&L.post_norm, H));
    if (d.has_qkv_bias) {
      ORION_TRY(alloc(&L.b_qkv, nqkv));
      ORION_CUDA_CHECK("clear bias", cudaMemsetAsync(L.b_qkv, 0, nqkv * sizeof(float), stream_));
    }
  }
  ORION_TRY(alloc(&embed_, V * H));
  ORION_TRY(alloc(&final_norm_, H));
  head_vn_ = d.vocab_size;
  if (d.tp_world > 1 && DTypeOf<T>::is_bf16 && gemm_plan(true, 1, 128, d.hidden_size, d.hidden_size, d.hidden_size).tensor_core) {
    const char *e = std::getenv("ORION_TP_VOCAB_PARALLEL");
    if (!e || std::atoi(e) != 0) {
      // column blocks in multiples of the 128-row weight tile; the last ranks may hold fewer (or no) rows
      const uint32_t per = ((d.vocab_size + d.tp_world - 1) / d.tp_world + 127) / 128 * 128;
      head_parallel_ = true;
      head_v0_ = std::min(d.vocab_size, d.tp_rank * per);
      head_vn_ = std::min(d.vocab_size, head_v0_ + per) - head_v0_;
    }
  }
  if (!d.tied_lm_head) ORION_TRY(alloc(&lm_head_own_, (size_t)head_vn_ * H));

  // Zero-initialised arena for this rank's KV heads (attention.rs:53-56).
  kv_ = KvLayout{d.num_layers, d.num_blocks, lkv_, d.block_size, d.head_dim,
                 (sizeof(T) == 2 && d.head_dim % 64 == 0) ? 1u : 0u};
  const size_t arena_elems = kv_.layer_elems() * d.num_layers;
  ORION_TRY(alloc(&arena_, arena_elems));
  ORION_CUDA_CHECK("clear arena", cudaMemsetAsync(arena_, 0, arena_elems * sizeof(T), stream_));

  // RopeTable::new (tensor.rs:228-253), same f32 recipe, computed on the host.
  {
    const size_t half = hd / 2, n = (size_t)d.max_position_embeddings * half;
    std::vector<float> c(n ? n : 1), s(n ? n : 1);
    for (size_t pos = 0; pos < d.max_position_embeddings; ++pos)
      for (size_t i = 0; i < half; ++i) {
        const float inv_freq = 1.0f / powf(d.rope_theta, 2.0f * (float)i / (float)hd);
        const float angle = (float)pos * inv_freq;
        c[pos * half + i] = cosf(angle);
        s[pos * half + i] = sinf(angle);
      }
    ORION_TRY(alloc(&rope_cos_, n));
    ORION_TRY(alloc(&rope_sin_, n));
    ORION_CUDA_CHECK("upload rope", cudaMemcpy(rope_cos_, c.data(), n * sizeof(float), cudaMemcpyHostToDevice));
    ORION_CUDA_CHECK("upload rope", cudaMemcpy(rope_sin_, s.data(), n * sizeof(float), cudaMemcpyHostToDevice));
  }

  // Work buffers sized for the largest batch.
  const size_t Tm = d.max_batch_tokens, Sm = d.max_batch_sequences;
  constexpr bool kBf16 = DTypeOf<T>::is_bf16;
  ORION_TRY(alloc(&hidden_, Tm * H));
  ORION_TRY(alloc(&normed_, Tm * H));
  ORION_TRY(alloc(&qbuf_, Tm * lq_ * hd));
  ORION_TRY(alloc(&attn_, Tm * lq_ * hd));
  ORION_TRY(alloc(&act_, Tm * lf_));
  ORION_TRY(alloc(&tail_, Sm * H));
  ORION_TRY(alloc(&logits_, Sm * V));
  ORION_TRY(alloc(&argmax_, Sm));
  partial_floats_ = gemm_partial_floats(kBf16, (uint32_t)Tm, (uint32_t)nqkv, (uint32_t)H);
  partial_floats_ = std::max(partial_floats_, gemm_partial_floats(kBf16, (uint32_t)Tm, (uint32_t)H, (uint32_t)(lq_ * hd)));
  partial_floats_ = std::max(partial_floats_, gemm_partial_floats(kBf16, (uint32_t)Tm, 2 * lf_, (uint32_t)H));
  partial_floats_ = std::max(partial_floats_, gemm_partial_floats(kBf16, (uint32_t)Tm, (uint32_t)H, lf_));
  ORION_TRY(alloc(&partial_, partial_floats_));
  ORION_TRY(alloc(&ready_, 1));
  ORION_CUDA_CHECK("clear ready counter", cudaMemsetAsync(ready_, 0, sizeof(uint32_t), stream_));
  if (kBf16 && decode_attention_supported(kv_, lq_)) {
    for (uint32_t r = 1; r <= Sm; ++r) {
      // room for the uniform split of r equally long rows, and for up to eight pieces of the long
      // rows of a ragged batch (a plan that wants more is cut back to what fits)
      const uint32_t s = std::max(decode_choose_splits(r, lkv_, d.max_position_embeddings, d.block_size, 32), 8u);
      dscratch_floats_ = std::max(dscratch_floats_, decode_scratch_floats(r, lq_, d.head_dim, s));
    }
    ORION_TRY(alloc(&dscratch_, dscratch_floats_));
    ORION_CUDA_CHECK("clear attention scratch", cudaMemsetAsync(dscratch_, 0, dscratch_floats_ * sizeof(float), stream_));
  }

  if (d.tp_world > 1) {
    nccl_.reset(new NcclCollective());
    ORION_TRY(nccl_->init(d.nccl_unique_id, (int)d.tp_rank, (int)d.tp_world));
    // Peer-memory hand-over (one kernel: all-reduce + residual + norm): one-shot at 2 ranks (every
    // partial sum to the peer: 4.01 vs 4.53 ms per headline step through NCCL), two-shot beyond
    // (one-shot is bandwidth-bound there: 4.29 vs 3.98 ms at 4 ranks, 6.10 vs 4.09 ms at 8).
    // ORION_TP_ALLREDUCE=fused / nccl forces either path; twoshot = fused, with the two-shot kernel
    // at 2 ranks as well (so that a 2-GPU machine can exercise it).
    const char *mode = std::getenv("ORION_TP_ALLREDUCE");
    const bool want_fused = mode ? (!strcmp(mode, "fused") || !strcmp(mode, "twoshot")) : true;
    tp_two_shot_ = d.tp_world > 2 || (mode && !strcmp(mode, "twoshot"));
    if (want_fused && d.tp_world <= (uint32_t)kMaxTpWorld && H % 4 == 0 && H / 4 <= 4096)
      ORION_TRY(setup_peer_handover());
    if (head_parallel_) ORION_TRY(setup_head_peers());
  }
  ORION_CUDA_CHECK("model init", cudaStreamSynchronize(stream_));
  return ORION_OK;
}

// Maps every rank's inbox into this process (CUDA IPC; the 64-byte handles travel through
// one NCCL all-gather) so that the fused all-reduce + residual + norm kernel can push its
// partial sums straight into the peers' memory.
template <typename T>
int Model<T>::setup_peer_handover() {
  const int world = (int)d_.tp_world, rank = (int)d_.tp_rank;
  const size_t slot_floats = (size_t)std::min(d_.max_batch_tokens, kTpFusedMaxRows) * d_.hidden_size;
  const size_t inbox_words = (2 * (size_t)world + 2) * slot_floats * 2;  // reduce-scatter slots + all-gather slots
  ORION_TRY(alloc(&tp_inbox_, inbox_words));
  ORION_CUDA_CHECK("clear inbox", cudaMemset(tp_inbox_, 0, inbox_words * sizeof(uint32_t)));  // epoch 0 is never sent
  constexpr int kFloatsPerHandle = sizeof(cudaIpcMemHandle_t) / sizeof(float);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  cudaIpcMemHandle_t mine;
  ORION_CUDA_CHECK("ipc export", cudaIpcGetMemHandle(&mine, tp_inbox_));
  float *d_send = nullptr, *d_recv = nullptr;
  ORION_TRY(alloc(&d_send, kFloatsPerHandle));
  ORION_TRY(alloc(&d_recv, (size_t)kFloatsPerHandle * world));
  ORION_CUDA_CHECK("ipc exchange", cudaMemcpy(d_send, &mine, sizeof mine, cudaMemcpyHostToDevice));
  ORION_TRY(nccl_->all_gather(d_send, d_recv, kFloatsPerHandle, stream_));
  ORION_TRY(nccl_->wait_stream(stream_, "ipc exchange"));
  std::vector<cudaIpcMemHandle_t> all((size_t)world);
  ORION_CUDA_CHECK("ipc exchange", cudaMemcpy(all.data(), d_recv, all.size() * sizeof(cudaIpcMemHandle_t),
                                               cudaMemcpyDeviceToHost));
  peers_.rank = rank;
  peers_.world = world;
  peers_.slot_floats = (uint32_t)slot_floats;
  for (int r = 0; r < world; ++r) {
    void *p = tp_inbox_;
    if (r != rank) {
      ORION_CUDA_CHECK("ipc import", cudaIpcOpenMemHandle(&p, all[(size_t)r], cudaIpcMemLazyEnablePeerAccess));
      ipc_opened_.push_back(p);
    }
    peers_.inbox[r] = static_cast<uint32_t *>(p);
  }
  ORION_TRY(alloc(&tp_state_, 2));
  const uint32_t first[2] = {1u, 0u};  // epoch 0 is never sent; the ready counter starts at zero
  ORION_CUDA_CHECK("hand-over state", cudaMemcpy(tp_state_, first, sizeof first, cudaMemcpyHostToDevice));
  ORION_TRY(nccl_->barrier(stream_));  // nobody starts a step before every mapping exists
  tp_fused_ = true;
  return ORION_OK;
}

// Maps the leader's logits buffer and flag words into every rank (CUDA IPC, handles over one NCCL
// all-gather) for the vocabulary-parallel LM head.
template <typename T>
int Model<T>::setup_head_peers() {
  const int world = (int)d_.tp_world, rank = (int)d_.tp_rank;
  uint32_t *flags = nullptr;
  ORION_TRY(alloc(&flags, 64));
  ORION_CUDA_CHECK("clear flags", cudaMemset(flags, 0, 64 * sizeof(uint32_t)));  // epoch 0 is never signalled
  constexpr int kFloatsPerHandle = sizeof(cudaIpcMemHandle_t) / sizeof(float);
  cudaIpcMemHandle_t mine[2];
  ORION_CUDA_CHECK("ipc export", cudaIpcGetMemHandle(&mine[0], logits_));
  ORION_CUDA_CHECK("ipc export", cudaIpcGetMemHandle(&mine[1], flags));
  float *d_send = nullptr, *d_recv = nullptr;
  ORION_TRY(alloc(&d_send, 2 * kFloatsPerHandle));
  ORION_TRY(alloc(&d_recv, (size_t)2 * kFloatsPerHandle * world));
  ORION_CUDA_CHECK("ipc exchange", cudaMemcpy(d_send, mine, sizeof mine, cudaMemcpyHostToDevice));
  ORION_TRY(nccl_->all_gather(d_send, d_recv, 2 * kFloatsPerHandle, stream_));
  ORION_TRY(nccl_->wait_stream(stream_, "ipc exchange"));
  cudaIpcMemHandle_t leader[2];
  ORION_CUDA_CHECK("ipc exchange", cudaMemcpy(leader, d_recv, sizeof leader, cudaMemcpyDeviceToHost));  // rank 0's pair comes first
  head_out_ = logits_;
  head_flags_ = flags;
  if (rank != 0) {
    void *p = nullptr;
    ORION_CUDA_CHECK("ipc import", cudaIpcOpenMemHandle(&p, leader[0], cudaIpcMemLazyEnablePeerAccess));
    ipc_opened_.push_back(p);
    head_out_ = static_cast<float *>(p);
    ORION_CUDA_CHECK("ipc import", cudaIpcOpenMemHandle(&p, leader[1], cudaIpcMemLazyEnablePeerAccess));
    ipc_opened_.push_back(p);
    head_flags_ = static_cast<uint32_t *>(p);
  }
  return nccl_->barrier(stream_);  // nobody starts a step before every mapping exists
}

template <typename T>
int Model<T>::upload_slice(T *dst_t, float *dst_f, const void *src, int dtype, uint64_t C,
                           uint64_t r0, uint64_t r1, uint64_t c0, uint64_t c1) {
  const size_t es = dtype_size(dtype);
  const uint64_t rows = r1 - r0, cols = c1 - c0;
  if (rows == 0 || cols == 0) return ORION_OK;
  const bool direct = dst_t ? (dtype == DTypeOf<T>::value) : (dtype == ORION_DTYPE_F32);
  const size_t row_bytes = cols * es;
  uint64_t chunk_rows = std::max<uint64_t>(1, (64ull << 20) / std::max<size_t>(row_bytes, 1));
  for (uint64_t r = 0; r < rows; r += chunk_rows) {
    const uint64_t nr = std::min(chunk_rows, rows - r);
    const uint8_t *s = static_cast<const uint8_t *>(src) + ((r0 + r) * C + c0) * es;
    const size_t n = nr * cols;
    void *direct_dst = dst_t ? static_cast<void *>(dst_t + r * cols) : static_cast<void *>(dst_f + r * cols);
    if (direct) {
      ORION_CUDA_CHECK("upload tensor", cudaMemcpy2DAsync(direct_dst, row_bytes, s, C * es, row_bytes, nr,
                                                          cudaMemcpyHostToDevice, stream_));
      ORION_CUDA_CHECK("upload tensor", cudaStreamSynchronize(stream_));
      continue;
    }
    ORION_TRY(ensure_stage(&stage_raw_, &stage_raw_cap_, n * es));
    ORION_CUDA_CHECK("upload tensor", cudaMemcpy2DAsync(stage_raw_, row_bytes, s, C * es, row_bytes, nr,
                                                        cudaMemcpyHostToDevice, stream_));
    // widen to f32 unless the source already is
    const float *as_f32 = nullptr;
    if (dtype == ORION_DTYPE_F32) {
      as_f32 = static_cast<const float *>(stage_raw_);
    } else {
      float *wide = nullptr;
      if (dst_f) {
        wide = dst_f + r * cols;
      } else {
        ORION_TRY(ensure_stage(&stage_f32_, &stage_f32_cap_, n * sizeof(float)));
        wide = static_cast<float *>(stage_f32_);
      }
      if (dtype == ORION_DTYPE_BF16)
        ORION_TRY(launch_convert_to_f32<bf16>(static_cast<const bf16 *>(stage_raw_), wide, n, stream_));
      else
        ORION_TRY(launch_f16_to_f32(static_cast<const uint16_t *>(stage_raw_), wide, n, stream_));
      as_f32 = wide;
    }
    if (dst_t) ORION_TRY(launch_convert_from_f32<T>(as_f32, dst_t + r * cols, n, stream_));
    ORION_CUDA_CHECK("upload tensor", cudaStreamSynchronize(stream_));
  }
  return ORION_OK;
}

template <typename T>
int Model<T>::load_tensor(const char *name, int dtype, const uint64_t *shape, int ndim,
                          const void *data) {
  const OrionModelDesc &d = d_;
  ORION_CUDA_CHECK("set device", cudaSetDevice(ordinal_));
  if (dtype_size(dtype) == 0 || dtype == ORION_DTYPE_I8 || dtype == ORION_DTYPE_I4)
    return set_error(ORION_ERR_MODEL, "unsupported dtype %d (tensor `%s`)", dtype, name);  // loader.rs:89-93
  if (!data || ndim < 1 || ndim > 2) return set_error(ORION_ERR_MODEL, "tensor `%s` has rank %d", name, ndim);
  const uint64_t R = ndim == 2 ? shape[0] : 1, C = ndim == 2 ? shape[1] : shape[0];
  const uint64_t H = d.hidden_size, hd = d.head_dim, V = d.vocab_size, F = d.ffn_dim;
  const uint64_t qd = (uint64_t)d.num_attention_heads * hd, kvd = (uint64_t)d.num_kv_heads * hd;
  auto expect = [&](uint64_t er, uint64_t ec) -> int {
    if (R != er || C != ec)
      return set_error(ORION_ERR_MODEL, "tensor `%s` has shape [%llu, %llu], expected [%llu, %llu]", name,
                       (unsigned long long)R, (unsigned long long)C, (unsigned long long)er,
                       (unsigned long long)ec);
    return ORION_OK;
  };
  const uint64_t q0 = lay_.query_heads.start * hd, q1 = q0 + lq_ * hd;
  const uint64_t k0 = lay_.kv_heads.start * hd, k1 = k0 + lkv_ * hd;
  const uint64_t f0 = lay_.ffn.start, f1 = f0 + lf_;
  finalized_ = false;

  if (!strcmp(name, "model.embed_tokens.weight")) {
    ORION_TRY(expect(V, H));
    got_embed_ = true;
    return upload_slice(embed_, nullptr, data, dtype, C, 0, V, 0, H);
  }
  if (!strcmp(name, "model.norm.weight")) {
    ORION_TRY(expect(1, H));
    got_final_norm_ = true;
    return upload_slice(nullptr, final_norm_, data, dtype, C, 0, 1, 0, H);
  }
  if (!strcmp(name, "lm_head.weight")) {
    if (d.tied_lm_head) return ORION_OK;  // transformer.rs:108-110
    ORION_TRY(expect(V, H));
    got_head_ = true;
    return upload_slice(lm_head_own_, nullptr, data, dtype, C, head_v0_, head_v0_ + head_vn_, 0, H);
  }
  unsigned li = 0;
  char rest[96];
  if (sscanf(name, "model.layers.%u.%95s", &li, rest) == 2 && li < d.num_layers) {
    Layer &L = layers_[li];
    const size_t lqd = (size_t)lq_ * hd, lkvd = (size_t)lkv_ * hd;
    if (!strcmp(rest, "input_layernorm.weight")) {
      ORION_TRY(expect(1, H));
      L.got |= kGotInNorm;
      return upload_slice(nullptr, L.in_norm, data, dtype, C, 0, 1, 0, H);
    }
    if (!strcmp(rest, "post_attention_layernorm.weight")) {
      ORION_TRY(expect(1, H));
      L.got |= kGotPostNorm;
      return upload_slice(nullptr, L.post_norm, data, dtype, C, 0, 1, 0, H);
    }
    if (!strcmp(rest, "self_attn.q_proj.weight")) {  // column-parallel: this rank's query heads
      ORION_TRY(expect(qd, H));
      L.got |= kGotQ;
      return upload_slice(L.w_qkv, nullptr, data, dtype, C, q0, q1, 0, H);
    }
    if (!strcmp(rest, "self_attn.k_proj.weight")) {
      ORION_TRY(expect(kvd, H));
      L.got |= kGotK;
      return upload_slice(L.w_qkv + lqd * H, nullptr, data, dtype, C, k0, k1, 0, H);
    }
    if (!strcmp(rest, "self_attn.v_proj.weight")) {
      ORION_TRY(expect(kvd, H));
      L.got |= kGotV;
      return upload_slice(L.w_qkv + (lqd + lkvd) * H, nullptr, data, dtype, C, k0, k1, 0, H);
    }
    if (!strcmp(rest, "self_attn.o_proj.weight")) {  // row-parallel: columns of this rank's heads
      ORION_TRY(expect(H, qd));
      L.got |= kGotO;
      return upload_slice(L.w_o, nullptr, data, dtype, C, 0, H, q0, q1);
    }
    const bool is_gate = !strcmp(rest, "mlp.gate_proj.weight");
    if (is_gate || !strcmp(rest, "mlp.up_proj.weight")) {
      ORION_TRY(expect(F, H));
      L.got |= is_gate ? kGotGate : kGotUp;
      if (!kInterleaveGateUp) return upload_slice(L.w_gu + (is_gate ? 0 : (size_t)lf_ * H), nullptr, data, dtype, C, f0, f1, 0, H);
      // gate row f -> row 2f, up row f -> row 2f + 1 (the GEMM epilogue pairs neighbouring rows)
      if (!gu_stage_) ORION_TRY(alloc(&gu_stage_, (size_t)lf_ * H));
      ORION_TRY(upload_slice(gu_stage_, nullptr, data, dtype, C, f0, f1, 0, H));
      ORION_TRY(launch_copy_rows_strided<T>(gu_stage_, L.w_gu + (is_gate ? 0 : H), lf_, H, 2 * (size_t)H, stream_));
      ORION_CUDA_CHECK("upload tensor", cudaStreamSynchronize(stream_));
      return ORION_OK;
    }
    if (!strcmp(rest, "mlp.down_proj.weight")) {
      ORION_TRY(expect(H, F));
      L.got |= kGotDown;
      return upload_slice(L.w_down, nullptr, data, dtype, C, 0, H, f0, f1);
    }
    const bool is_bias = !strcmp(rest, "self_attn.q_proj.bias") || !strcmp(rest, "self_attn.k_proj.bias") ||
                         !strcmp(rest, "self_attn.v_proj.bias");
    if (is_bias) {
      if (!d.has_qkv_bias) return ORION_OK;  // transformer.rs:84-86: Llama never reads biases
      const char which = rest[10];
      if (which == 'q') {
        ORION_TRY(expect(1, qd));
        return upload_slice(nullptr, L.b_qkv, data, dtype, C, 0, 1, q0, q1);
      }
      ORION_TRY(expect(1, kvd));
      float *dst = L.b_qkv + lqd + (which == 'v' ? lkvd : 0);
      return upload_slice(nullptr, dst, data, dtype, C, 0, 1, k0, k1);
    }
  }
  return set_error(ORION_ERR_MODEL, "tensor `%s` is not part of the Llama/Qwen2 layout", name);
}

template <typename T>
int Model<T>::init_random(uint64_t seed, float std) {
  // N(0, std) matrices, RMSNorm weights 1.0, zero biases. Values are drawn on
  // the device; they depend on (seed, tensor index) only.
  const OrionModelDesc &d = d_;
  ORION_CUDA_CHECK("set device", cudaSetDevice(ordinal_));
  const size_t H = d.hidden_size, hd = d.head_dim, V = d.vocab_size;
  uint64_t tensor = 0;
  auto fill = [&](T *p, size_t n) -> int {
    ORION_TRY(ensure_stage(&stage_f32_, &stage_f32_cap_, std::min<size_t>(n, 64u << 20) * sizeof(float)));
    for (size_t off = 0; off < n; off += (64u << 20)) {
      const size_t m = std::min<size_t>(64u << 20, n - off);
      float *tmp = static_cast<float *>(stage_f32_);
      ORION_TRY(launch_fill_normal<float>(tmp, m, seed * 0x9E3779B97F4A7C15ull + (++tensor), stream_));
      ORION_TRY(launch_scale_convert<T>(tmp, p + off, m, std, stream_));  // N(0,1) -> N(0,std), narrowed to T
    }
    return ORION_OK;
  };
  std::vector<float> ones(H, 1.0f);
  auto set_ones = [&](float *p) -> int {
    ORION_CUDA_CHECK("init norm", cudaMemcpyAsync(p, ones.data(), H * sizeof(float), cudaMemcpyHostToDevice, stream_));
    return ORION_OK;
  };
  ORION_TRY(fill(embed_, V * H));
  if (lm_head_own_) ORION_TRY(fill(lm_head_own_, (size_t)head_vn_ * H));
  ORION_TRY(set_ones(final_norm_));
  for (Layer &L : layers_) {
    ORION_TRY(fill(L.w_qkv, (size_t)(lq_ + 2 * lkv_) * hd * H));
    ORION_TRY(fill(L.w_o, H * lq_ * hd));
    ORION_TRY(fill(L.w_gu, (size_t)2 * lf_ * H));
    ORION_TRY(fill(L.w_down, H * lf_));
    ORION_TRY(set_ones(L.in_norm));
    ORION_TRY(set_ones(L.post_norm));
    L.got = kGotAllLayer;
  }
  got_embed_ = got_final_norm_ = true;
  got_head_ = lm_head_own_ != nullptr;
  ORION_CUDA_CHECK("init_random", cudaStreamSynchronize(stream_));
  return finalize();
}

template <typename T>
int Model<T>::finalize() {
  // ModelWeights::load fails on the first missing tensor (transformer.rs:73-118).
  if (!got_embed_) return set_error(ORION_ERR_MODEL, "missing tensor `model.embed_tokens.weight`");
  if (!got_final_norm_) return set_error(ORION_ERR_MODEL, "missing tensor `model.norm.weight`");
  static const char *names[] = {"input_layernorm.weight", "post_attention_layernorm.weight",
                                "self_attn.q_proj.weight", "self_attn.k_proj.weight",
                                "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                                "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight"};
  for (size_t i = 0; i < layers_.size(); ++i)
    for (int b = 0; b < 9; ++b)
      if (!(layers_[i].got & (1u << b)))
        return set_error(ORION_ERR_MODEL, "missing tensor `model.layers.%zu.%s`", i, names[b]);
  // transformer.rs:108-112: the head falls back to the embedding when tied or absent.
  lm_head_ = (d_.tied_lm_head || !got_head_) ? embed_ + (size_t)head_v0_ * d_.hidden_size : lm_head_own_;
  finalized_ = true;
  return ORION_OK;
}

template <typename T>
int Model<T>::tp_reduce(uint32_t *splits, size_t slab) {
  if (!nccl_) return ORION_OK;
  // Row-parallel projection: sum this rank's split-K slabs, then the one
  // all-reduce of the half-layer (orion-distributed/src/lib.rs:317-319).
  if (*splits > 1) ORION_TRY(launch_finish_linear(partial_, *splits, slab, nullptr, partial_, 1, (uint32_t)slab, stream_));
  *splits = 1;
  return nccl_->all_reduce_sum(partial_, slab, stream_);
}

template <typename T>
int Model<T>::handover(uint32_t splits, const float *norm_w, T *out, const uint32_t *row_map, uint32_t out_rows, bool count_ready) {
  const uint32_t Tn = meta_.rows, H = d_.hidden_size;
  const size_t slab = (size_t)Tn * H;
  if (nccl_ && tp_fused_ && Tn <= kTpFusedMaxRows) {
    // every rank ends up with the whole residual stream and all Tn normalised rows
    ORION_TRY(launch_tp_allreduce_residual_rmsnorm<T>(peers_, tp_state_, step_epochs_, partial_, splits, slab, hidden_, norm_w,
                                                      d_.rms_norm_eps, normed_, Tn, H,
                                                      // at 2 ranks the one-shot kernel wins while the payload is small; from
                                                      // 1 Mi elements on (128 rows x 8192) the two-shot kernel with its bf16
                                                      // units moves a quarter of the bytes and measured 6 % faster per step
                                                      tp_two_shot_ || (sizeof(T) == 2 && (size_t)Tn * H >= ((size_t)1 << 20)),
                                                      stream_, count_ready && !row_map ? ready_ : nullptr));
    if (count_ready && !row_map) step_rows_counted_ += Tn;
    ++step_epochs_;
    if (row_map) return launch_gather_rows<T>(normed_, row_map, out, out_rows, H, stream_);
    if (out != normed_) return set_error(ORION_ERR_INTERNAL, "fused hand-over writes the activation buffer only");
    return ORION_OK;
  }
  ORION_TRY(tp_reduce(&splits, slab));
  ORION_TRY(launch_residual_rmsnorm<T>(partial_, splits, slab, hidden_, norm_w, d_.rms_norm_eps, out, row_map, out_rows, H,
                                       stream_, count_ready ? ready_ : nullptr));
  if (count_ready) step_rows_counted_ += out_rows;
  return ORION_OK;
}

template <typename T>
int Model<T>::run_step_graphed(bool want_argmax) {
  const GraphKey key = layout_key();
  key_streak_ = (key_streak_ > 0 && key == last_key_) ? key_streak_ + 1 : 1;
  last_key_ = key;
  auto it = graphs_.find(key);
  if (it == graphs_.end() && key_streak_ >= kGraphAfterSteps) {
    if (graphs_.size() >= kMaxStepGraphs) drop_graphs();
    cudaGraph_t graph = nullptr;
    StepGraph sg;  // stays without an executable graph if anything below fails: the layout is then launched kernel by kernel
    const uint64_t before = g_launch_count;
    if (cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
      const int rc = run_step_body(false, 1);
      const cudaError_t ce = cudaStreamEndCapture(stream_, &graph);
      sg.launches = g_launch_count - before;
      if (rc != ORION_OK || ce != cudaSuccess || cudaGraphInstantiate(&sg.exec, graph, 0) != cudaSuccess) sg.exec = nullptr;
      if (graph) cudaGraphDestroy(graph);
    }
    g_launch_count = before;
    if (!sg.exec) {
      cudaGetLastError();  // the failed capture's error is not the step's
      clear_error();
    }
    it = graphs_.emplace(key, sg).first;
  }
  if (it != graphs_.end() && it->second.exec) {
    ORION_CUDA_CHECK("step graph launch", cudaGraphLaunch(it->second.exec, stream_));
    g_launch_count += it->second.launches;
  } else {
    ORION_TRY(run_step_body(want_argmax, 1));
  }
  return run_step_body(want_argmax, 2);
}

template <typename T>
int Model<T>::run_step_body(bool want_argmax, int part) {
  const OrionModelDesc &d = d_;
  constexpr bool kBf16 = DTypeOf<T>::is_bf16;
  const uint32_t Tn = meta_.rows, S = meta_.seqs, H = d.hidden_size, hd = d.head_dim;
  const uint32_t nqkv = (lq_ + 2 * lkv_) * hd, qd = lq_ * hd;
  const uint32_t *m = d_meta_;
  const uint32_t *tokens = m + meta_.tokens, *positions = m + meta_.positions;
  const uint32_t *slot_block = m + meta_.slot_block, *slot_slot = m + meta_.slot_slot;
  const uint32_t *last_rows = m + meta_.last_rows;
  AttnBatch ab{positions, m + meta_.seq_of_row, m + meta_.tables, m + meta_.offsets, Tn, meta_.max_position};
  const bool tuned_decode = kBf16 && meta_.decode && decode_attention_supported(kv_, lq_);
  // The work buffers were sized at creation under the tuning values of that moment; a tuning call
  // made since may ask for more k splits or context splits than they hold, so every plan is cut
  // back to the capacity before it is launched.
  auto fit_context_splits = [&](uint32_t rows, uint32_t want) {
    while (want > 1 && decode_scratch_floats(rows, lq_, hd, want) > dscratch_floats_) --want;
    return want;
  };
  auto plan_for = [&](uint32_t rows, uint32_t n, uint32_t k) {
    GemmPlan p = gemm_plan(kBf16, rows, n, k, k, k);
    while (p.splits > 1 && (size_t)p.splits * rows * n > partial_floats_) {
      --p.splits;
      if (!p.cluster_reduce) p.out_slabs = p.splits;
    }
    if (p.splits == 1) p.cluster_reduce = false, p.out_slabs = 1;
    return p;
  };
  const DecodePlan dplan = tuned_decode ? decode_plan(Tn, lkv_, meta_.total_blocks, meta_.max_position, d.block_size, 32)
                                        : DecodePlan{1, 0};
  const uint32_t dsplits = fit_context_splits(Tn, dplan.splits);
  // Under tensor parallelism the projection that follows a fused hand-over polls that kernel's count of finished
  // rows instead of waiting for its completion: a kernel that has stored to peer memory releases its dependents
  // about 3 us later than one that has not (measured 4.5 against 1.5 us), and the count does not wait for that
  // (3.33 -> 3.25 ms per step at 2 ranks). On one GPU the two are equally fast, so the counter is left out. Never
  // in a timing replay that leaves kernel families out, where the counting kernel may be missing.
  const bool count_ready = g_ready_counters && kBf16 && nccl_ && tp_fused_ && Tn <= kTpFusedMaxRows && only_mask_ == 0;
  if (tp_broken_)
    return set_error(ORION_ERR_BACKEND, "backend cuda failed at forward: an earlier tensor-parallel step ended half way; the model cannot continue");
  if (part != 2) step_epochs_ = step_rows_counted_ = 0;
  auto ready_for = [&](const GemmPlan &gp) {
    ReadyWait r;
    if (count_ready && gp.tensor_core) r.counter = ready_, r.target = step_rows_counted_, r.base = tp_state_ + 1;
    return r;
  };

  if (part != 2)
    ORION_TRY(timed(kProfElementwise, [&] { return launch_embed_rmsnorm<T>(embed_, tokens, layers_[0].in_norm, d.rms_norm_eps, hidden_, normed_, Tn, H, stream_); }));
  for (uint32_t l = 0; part != 2 && l < d.num_layers; ++l) {
    const Layer &L = layers_[l];
    GemmPlan p = plan_for(Tn, nqkv, H);
    // layer 0 follows the embedding kernel, which counts nothing
    ORION_TRY(timed(kProfGemm, [&] { return launch_gemm<T>(normed_, H, L.w_qkv, H, partial_, Tn, nqkv, H, p, stream_,
                                                              l > 0 ? ready_for(p) : ReadyWait{}); }));
    // Pure decode batches on the tuned path: the attention kernel folds the QKV partials, applies
    // RoPE and writes the KV slot itself, so the separate kernel (and its launch hop) is left out.
    const bool fuse_qkv = tuned_decode && g_fuse_qkv;
    if (!fuse_qkv)
      ORION_TRY(timed(kProfElementwise, [&] { return launch_rope_kvwrite<T>(partial_, p.out_slabs, (size_t)Tn * nqkv, L.b_qkv, positions, slot_block,
                                       slot_slot, rope_cos_, rope_sin_, qbuf_, arena_, kv_, l, Tn, lq_, stream_); }));
    if (tuned_decode) {
      if constexpr (kBf16) {
        DecodeScratch sc = decode_scratch_at(dscratch_, Tn, lq_, lkv_, hd, dsplits, dplan.blocks_per_split);
        FusedQkv fq;
        if (fuse_qkv) {
          fq.partial = partial_;
          fq.slabs = p.out_slabs;
          fq.slab_stride = (size_t)Tn * nqkv;
          fq.bias = L.b_qkv;
          fq.rope_cos = rope_cos_;
          fq.rope_sin = rope_sin_;
          fq.slot_block = slot_block;
          fq.arena = arena_;
        }
        ORION_TRY(timed(kProfAttention, [&] { return launch_paged_attention_decode(qbuf_, arena_, kv_, l, ab, lq_, dsplits, sc, attn_, stream_, fq); }));
      }
    } else if (meta_.num_tiles > 0 || meta_.dec_rows > 0) {
      if constexpr (kBf16) {
        if (meta_.dec_rows > 0) {  // the decode rows of a mixed batch: one contiguous run of rows
          const uint32_t r0 = meta_.dec_row0, n = meta_.dec_rows;
          AttnBatch sub{positions + r0, m + meta_.seq_of_row + r0, ab.tables_flat, ab.table_offsets, n, meta_.max_position};
          const uint32_t sp = fit_context_splits(n, decode_choose_splits(n, lkv_, meta_.max_position, d.block_size, 32));
          DecodeScratch sc = decode_scratch_at(dscratch_, n, lq_, lkv_, hd, sp);
          ORION_TRY(timed(kProfAttention, [&] { return launch_paged_attention_decode(qbuf_ + (size_t)r0 * qd, arena_, kv_, l, sub, lq_, sp, sc,
                                                                                       attn_ + (size_t)r0 * qd, stream_); }));
        }
        if (meta_.num_tiles > 0) {
          const PrefillTile *tiles = reinterpret_cast<const PrefillTile *>(m + meta_.tiles);
          ORION_TRY(timed(kProfAttention, [&] { return launch_paged_attention_prefill(qbuf_, arena_, kv_, l, ab, tiles, meta_.num_tiles, lq_, attn_, stream_); }));
        }
      }
    } else {
      ORION_TRY(timed(kProfAttention, [&] { return launch_paged_attention_generic<T>(qbuf_, arena_, kv_, l, ab, lq_, attn_, stream_); }));
    }
    p = plan_for(Tn, H, qd);
    ORION_TRY(timed(kProfGemm, [&] { return launch_gemm<T>(attn_, qd, L.w_o, qd, partial_, Tn, H, qd, p, stream_); }));
    const int handover_cat = nccl_ ? kProfCollective : kProfElementwise;
    ORION_TRY(timed(handover_cat, [&] { return handover(p.out_slabs, L.post_norm, normed_, nullptr, Tn, count_ready); }));
    p = plan_for(Tn, 2 * lf_, H);
    bool fused_swiglu = false;
    if constexpr (kBf16) {
      if (p.tensor_core && p.splits == 1 && g_fuse_swiglu) {  // SwiGLU in the GEMM epilogue: no partials, no extra launch
        fused_swiglu = true;
        ORION_TRY(timed(kProfGemm, [&] { return launch_gemm_swiglu(normed_, H, L.w_gu, H, act_, Tn, lf_, H, stream_, ready_for(p)); }));
      }
    }
    if (!fused_swiglu) {
      ORION_TRY(timed(kProfGemm, [&] { return launch_gemm<T>(normed_, H, L.w_gu, H, partial_, Tn, 2 * lf_, H, p, stream_, ready_for(p)); }));
      ORION_TRY(timed(kProfElementwise, [&] { return launch_swiglu<T>(partial_, p.out_slabs, (size_t)Tn * 2 * lf_, act_, Tn, lf_, stream_,
                                                                       kInterleaveGateUp); }));
    }
    p = plan_for(Tn, H, lf_);
    ORION_TRY(timed(kProfGemm, [&] { return launch_gemm<T>(act_, lf_, L.w_down, lf_, partial_, Tn, H, lf_, p, stream_); }));
    if (l + 1 < d.num_layers) {
      ORION_TRY(timed(handover_cat, [&] { return handover(p.out_slabs, layers_[l + 1].in_norm, normed_, nullptr, Tn, count_ready); }));
    } else if (!meta_.zero_count) {
      // Final norm over the last row of every sequence (transformer.rs:401-428;
      // the norm is row-wise, so gathering first gives the same rows).
      ORION_TRY(timed(handover_cat, [&] { return handover(p.out_slabs, final_norm_, tail_, last_rows, S); }));
    } else if (nccl_) {
      // keep the ranks in lock step even though this step ends in an error
      ORION_TRY(timed(handover_cat, [&] { return handover(p.out_slabs, final_norm_, normed_, nullptr, Tn); }));
    }
  }
  if (part != 2 && step_epochs_ > 0)  // the device state moves on to the next step
    ORION_TRY(timed(kProfCollective, [&] { return launch_tp_state_bump(tp_state_, step_epochs_, step_rows_counted_, stream_); }));
  if (part == 1 || meta_.zero_count) return ORION_OK;
  if (head_parallel_) {
    // This rank's column block of the logits goes straight into the leader's buffer (plain peer stores from
    // the GEMM epilogue), then the rank raises its flag there; the leader waits for all flags.
    if (head_vn_ > 0) {
      GemmPlan hp = gemm_plan(kBf16, S, head_vn_, H, H, H);
      hp.splits = hp.out_slabs = 1, hp.cluster_reduce = false;
      hp.ldc = d.vocab_size;
      ORION_TRY(timed(kProfGemm, [&] { return launch_gemm<T>(tail_, H, lm_head_, H, head_out_ + head_v0_, S, head_vn_, H, hp, stream_); }));
    }
    head_chunks_ = 0;
    const uint32_t epoch = head_epoch_;
    head_epoch_ = head_epoch_ == 0xFFFFFFFEu ? 1u : head_epoch_ + 1;
    if (d.tp_rank != 0)
      return timed(kProfCollective, [&] { return launch_tp_signal(head_flags_ + d.tp_rank, epoch, stream_); });
    ORION_TRY(timed(kProfCollective, [&] { return launch_tp_wait_flags(head_flags_, epoch, (int)d.tp_world, 2000000000ull, stream_); }));
    if (want_argmax) ORION_TRY(timed(kProfElementwise, [&] { return launch_argmax(logits_, S, d.vocab_size, argmax_, stream_); }));
    return ORION_OK;
  }
  GemmPlan hp = gemm_plan(kBf16, S, d.vocab_size, H, H, H);
  hp.splits = hp.out_slabs = 1, hp.cluster_reduce = false;  // logits are written in place, row-major [S][V]
  head_chunks_ = 0;
  if (kBf16 && hp.tensor_core && d.vocab_size >= 4 * 8192 && !want_argmax) {
    // A large vocabulary goes out in column blocks, an event after each: forward() copies block i
    // to the host (copy engine, second stream) while block i + 1 is being computed.
    const uint32_t per = (((d.vocab_size + 127) / 128 + kHeadChunks - 1) / kHeadChunks) * 128;
    for (uint32_t c = 0; c < (uint32_t)kHeadChunks && c * per < d.vocab_size; ++c) {
      const uint32_t n0 = c * per, nn = std::min(per, d.vocab_size - n0);
      GemmPlan cp = hp;
      cp.ldc = d.vocab_size;
      ORION_TRY(timed(kProfGemm, [&] { return launch_gemm<T>(tail_, H, lm_head_ + (size_t)n0 * H, H, logits_ + n0, S, nn, H, cp, stream_); }));
      ORION_CUDA_CHECK("lm head", cudaEventRecord(head_ev_[c], stream_));
      head_off_[c] = n0;
      head_cols_[c] = nn;
      head_chunks_ = c + 1;
    }
    return ORION_OK;
  }
  ORION_TRY(timed(kProfGemm, [&] { return launch_gemm<T>(tail_, H, lm_head_, H, logits_, S, d.vocab_size, H, hp, stream_); }));
  if (want_argmax) ORION_TRY(timed(kProfElementwise, [&] { return launch_argmax(logits_, S, d.vocab_size, argmax_, stream_); }));
  return ORION_OK;
}

template <typename T>
int Model<T>::forward(const BatchView &b, float *logits_out, uint64_t logits_capacity,
                      uint32_t *token_ids_out) {
  const OrionModelDesc &d = d_;
  if (!finalized_) return set_error(ORION_ERR_MODEL, "model weights are not finalized");
  // ForwardBatch::validate (orion-core/src/traits.rs:232-261)
  const uint64_t S = b.num_sequences;
  if (b.num_slot_token_counts != S || b.num_context_lens != S || b.num_block_tables != S)
    return set_error(ORION_ERR_INTERNAL,
                     "ForwardBatch arrays disagree: %llu sequence ids, %llu token counts, %llu context "
                     "lens, %llu block tables",
                     (unsigned long long)S, (unsigned long long)b.num_slot_token_counts,
                     (unsigned long long)b.num_context_lens, (unsigned long long)b.num_block_tables);
  if (b.num_positions != b.num_tokens)
    return set_error(ORION_ERR_INTERNAL, "ForwardBatch has %llu tokens but %llu positions",
                     (unsigned long long)b.num_tokens, (unsigned long long)b.num_positions);
  // Malformed calls across the C boundary (the Rust vectors cannot be null or out of order).
  if ((b.num_tokens > 0 && (!b.tokens || !b.positions)) || (S > 0 && (!b.slot_token_counts || !b.block_table_offsets)))
    return set_error(ORION_ERR_INVALID_REQUEST, "null batch array");
  for (uint64_t s = 0; s < S; ++s)
    if (b.block_table_offsets[s + 1] < b.block_table_offsets[s])
      return set_error(ORION_ERR_INVALID_REQUEST, "block table offsets decrease at sequence %llu", (unsigned long long)s);
  if (S > 0 && b.block_table_offsets[S] > 0 && !b.block_tables_flat)
    return set_error(ORION_ERR_INVALID_REQUEST, "null batch array");
  uint64_t summed = 0;
  for (uint64_t s = 0; s < S; ++s) summed += b.slot_token_counts[s];
  if (summed != b.num_tokens)
    return set_error(ORION_ERR_INTERNAL,
                     "ForwardBatch slot token counts sum to %llu but there are %llu tokens",
                     (unsigned long long)summed, (unsigned long long)b.num_tokens);
  last_launches_ = 0;
  if (b.num_tokens == 0) return ORION_OK;  // transformer.rs:361-367: empty batch, empty output
  const uint64_t Tn = b.num_tokens;
  if (Tn > d.max_batch_tokens || S > d.max_batch_sequences)
    return set_error(ORION_ERR_INVALID_REQUEST,
                     "batch of %llu tokens / %llu sequences exceeds the configured capacity (%u / %u)",
                     (unsigned long long)Tn, (unsigned long long)S, d.max_batch_tokens,
                     d.max_batch_sequences);
  if (logits_out && logits_capacity < S * (uint64_t)d.vocab_size)
    return set_error(ORION_ERR_INVALID_REQUEST, "logits buffer holds %llu floats, %llu needed",
                     (unsigned long long)logits_capacity, (unsigned long long)(S * (uint64_t)d.vocab_size));

  ORION_CUDA_CHECK("set device", cudaSetDevice(ordinal_));
  const uint64_t table_entries = S ? b.block_table_offsets[S] : 0;
  Meta mt;
  mt.rows = (uint32_t)Tn;
  mt.seqs = (uint32_t)S;
  mt.tokens = 0;
  mt.positions = Tn;
  mt.slot_block = 2 * Tn;
  mt.slot_slot = 3 * Tn;
  mt.seq_of_row = 4 * Tn;
  mt.last_rows = 5 * Tn;
  mt.offsets = 5 * Tn + S;
  mt.tables = 5 * Tn + 2 * S + 1;
  mt.tiles = mt.tables + table_entries;
  constexpr bool kBf16Build = DTypeOf<T>::is_bf16;
  const bool tuned_prefill = kBf16Build && prefill_attention_supported(kv_, lq_);
  const uint32_t tile_rows = tuned_prefill ? prefill_tile_positions(lq_, lkv_) : 0;
  const size_t max_tiles = tile_rows ? S + Tn / tile_rows + 1 : 0;
  mt.total = mt.tiles + 4 * max_tiles;
  if (table_entries > UINT32_MAX) return set_error(ORION_ERR_INVALID_REQUEST, "block tables too large");
  if (mt.total > meta_cap_) {
    const size_t cap = mt.total * 2 + 1024;
    if (h_meta_) cudaFreeHost(h_meta_);
    h_meta_ = nullptr;
    meta_cap_ = 0;
    ORION_CUDA_CHECK("allocate batch mirror", cudaMallocHost(reinterpret_cast<void **>(&h_meta_), cap * sizeof(uint32_t)));
    ORION_TRY(alloc(&d_meta_, cap));  // the previous device array stays owned until destruction
    drop_graphs();                    // captured steps point into the previous array
    meta_cap_ = cap;
  }
  uint32_t *h = h_meta_;
  // seq_of_row and slot resolution BEFORE any compute or KV write (transformer.rs:371-387).
  {
    uint64_t row = 0;
    for (uint64_t s = 0; s < S; ++s) {
      for (uint64_t c = 0; c < b.slot_token_counts[s]; ++c) h[mt.seq_of_row + row++] = (uint32_t)s;
      if (b.slot_token_counts[s] == 0) mt.zero_count = true;
    }
  }
  const uint32_t B = d.block_size;
  bool all_single = true;
  for (uint64_t s = 0; s < S; ++s) all_single &= (b.slot_token_counts[s] == 1);
  for (uint64_t row = 0; row < Tn; ++row) {
    const uint32_t seq = h[mt.seq_of_row + row], pos = b.positions[row];
    const uint64_t t0 = b.block_table_offsets[seq], tlen = b.block_table_offsets[seq + 1] - t0;
    const uint64_t logical = pos / B;  // locate, attention.rs:182-186
    if (logical >= tlen)
      return set_error(ORION_ERR_INTERNAL, "position %u has no block in the table for sequence %u", pos, seq);
    h[mt.slot_block + row] = b.block_tables_flat[t0 + logical];
    h[mt.slot_slot + row] = pos % B;
    mt.max_position = std::max(mt.max_position, pos);
    mt.total_blocks += logical + 1;
  }
  for (uint64_t row = 0; row < Tn; ++row)  // embed, transformer.rs:211-217
    if (b.tokens[row] >= d.vocab_size)
      return set_error(ORION_ERR_INTERNAL, "token id %u is outside the vocabulary of %u", b.tokens[row],
                       d.vocab_size);
  for (uint64_t row = 0; row < Tn; ++row)  // RoPE range, transformer.rs:255-262
    if (b.positions[row] >= d.max_position_embeddings)
      return set_error(ORION_ERR_INTERNAL, "position %u exceeds the RoPE table (%u entries)", b.positions[row],
                       d.max_position_embeddings);
  // Every block a query row will read must exist in the arena (attention.rs:150-155);
  // checked here so that no kernel ever sees an out-of-range block id.
  for (uint64_t row = 0; row < Tn; ++row) {
    const uint32_t seq = h[mt.seq_of_row + row];
    const uint64_t t0 = b.block_table_offsets[seq];
    const uint64_t used = (uint64_t)b.positions[row] / B + 1;
    for (uint64_t e = 0; e < used; ++e)
      if (b.block_tables_flat[t0 + e] >= d.num_blocks)
        return set_error(ORION_ERR_INTERNAL, "block %u out of range (have %u)", b.block_tables_flat[t0 + e],
                         d.num_blocks);
  }
  std::memcpy(h + mt.tokens, b.tokens, Tn * sizeof(uint32_t));
  std::memcpy(h + mt.positions, b.positions, Tn * sizeof(uint32_t));
  {
    uint64_t cursor = 0;
    for (uint64_t s = 0; s < S; ++s) {  // transformer.rs:410-420
      cursor += b.slot_token_counts[s];
      h[mt.last_rows + s] = (uint32_t)(cursor ? cursor - 1 : 0);
      h[mt.offsets + s] = (uint32_t)b.block_table_offsets[s];
    }
    h[mt.offsets + S] = (uint32_t)table_entries;
  }
  if (table_entries) std::memcpy(h + mt.tables, b.block_tables_flat, table_entries * sizeof(uint32_t));
  mt.decode = all_single;
  if (tuned_prefill && !all_single) {
    if (decode_attention_supported(kv_, lq_)) {
      uint64_t head = 0, tail = 0;
      while (head < S && b.slot_token_counts[head] == 1) ++head;
      while (tail < S && b.slot_token_counts[S - 1 - tail] == 1) ++tail;
      if (std::max(head, tail) >= 8) {  // worth a launch of its own
        mt.dec_rows = (uint32_t)std::max(head, tail);
        mt.dec_row0 = head >= tail ? 0u : (uint32_t)(Tn - tail);
      }
    }
    // Tiles of consecutive rows of one sequence for the prefill attention kernel.
    uint32_t *t = h + mt.tiles;
    uint64_t row = 0;
    for (uint64_t s = 0; s < S; ++s) {
      const uint64_t end = row + b.slot_token_counts[s];
      if (row >= mt.dec_row0 && row < (uint64_t)mt.dec_row0 + mt.dec_rows) {  // a decode row: no tile
        row = end;
        continue;
      }
      while (row < end) {
        const uint32_t n = (uint32_t)std::min<uint64_t>(tile_rows, end - row);
        uint32_t max_pos = 0;
        for (uint32_t i = 0; i < n; ++i) max_pos = std::max(max_pos, b.positions[row + i]);
        t[0] = (uint32_t)row;
        t[1] = n;
        t[2] = (uint32_t)s;
        t[3] = max_pos;
        t += 4;
        ++mt.num_tiles;
        row += n;
      }
    }
  }
  meta_ = mt;

  g_launch_count = 0;
  ORION_CUDA_CHECK("upload batch", cudaMemcpyAsync(d_meta_, h, mt.total * sizeof(uint32_t), cudaMemcpyHostToDevice, stream_));
  ORION_TRY(run_step(token_ids_out != nullptr));
  last_launches_ = g_launch_count;
  if (mt.zero_count) {
    ORION_TRY(wait_for(stream_, "forward"));
    // transformer.rs:413-417: detected after the layers ran, so KV slots were written.
    return set_error(ORION_ERR_INTERNAL, "a scheduled sequence contributed zero tokens");
  }
  if (d.tp_world > 1 && d.tp_rank != 0) {  // only the leader returns logits (Rank::is_leader)
    ORION_TRY(wait_for(stream_, "forward"));
  } else {
    if (logits_out && head_chunks_ > 0) {
      const size_t pitch = (size_t)d.vocab_size * sizeof(float);
      for (int c = 0; c < head_chunks_; ++c) {  // block c leaves while the blocks after it are computed
        ORION_CUDA_CHECK("download logits", cudaStreamWaitEvent(copy_stream_, head_ev_[c], 0));
        ORION_CUDA_CHECK("download logits", cudaMemcpy2DAsync(logits_out + head_off_[c], pitch, logits_ + head_off_[c], pitch,
                                                              (size_t)head_cols_[c] * sizeof(float), S, cudaMemcpyDeviceToHost,
                                                              copy_stream_));
      }
      ORION_TRY(wait_for(copy_stream_, "download logits"));
    } else if (logits_out) {
      ORION_CUDA_CHECK("download logits", cudaMemcpyAsync(logits_out, logits_, S * (size_t)d.vocab_size * sizeof(float),
                                                          cudaMemcpyDeviceToHost, stream_));
    }
    if (token_ids_out)
      ORION_CUDA_CHECK("download tokens", cudaMemcpyAsync(token_ids_out, argmax_, S * sizeof(uint32_t),
                                                          cudaMemcpyDeviceToHost, stream_));
    ORION_TRY(wait_for(stream_, "forward"));
  }
  uint32_t code = 0;
  if (nccl_) {
    ORION_TRY(tp_poll_error(&code));
    if (code) return set_error(ORION_ERR_BACKEND, "backend cuda failed at all_reduce: a peer did not arrive within the wait limit (code %u)", code);
  }
  if (DTypeOf<T>::is_bf16) {
    ORION_TRY(gemm_tc_poll_error(&code));
    if (code) return set_error(ORION_ERR_BACKEND, "backend cuda failed at gemm: a bounded pipeline wait ran out (code %u)", code);
    ORION_TRY(prefill_poll_error(&code));
    if (code) return set_error(ORION_ERR_BACKEND, "backend cuda failed at prefill attention: a bounded pipeline wait ran out (code %u)", code);
    ORION_TRY(decode_poll_error(&code));
    if (code) return set_error(ORION_ERR_BACKEND, "backend cuda failed at attention: a bounded pipeline wait ran out (code %u)", code);
  }
  return ORION_OK;
}

template <typename T>
int Model<T>::replay(int iterations, uint32_t category_mask, float *elapsed_ms) {
  if (meta_.rows == 0 || meta_.zero_count)
    return set_error(ORION_ERR_INVALID_REQUEST, "replay needs a preceding successful forward");
  ORION_CUDA_CHECK("set device", cudaSetDevice(ordinal_));
  ORION_CUDA_CHECK("replay", cudaStreamSynchronize(stream_));
  only_mask_ = category_mask & ((1u << kProfCategories) - 1);
  // a layout that will be replayed as a graph is brought there before the clock starts
  for (uint32_t i = 0; i <= kGraphAfterSteps && graph_eligible() && graphs_.find(layout_key()) == graphs_.end(); ++i) {
    const int rc = run_step(false);
    if (rc != ORION_OK) {
      only_mask_ = 0;
      return rc;
    }
  }
  ORION_CUDA_CHECK("replay", cudaEventRecord(ev0_, stream_));
  for (int i = 0; i < iterations; ++i) {
    g_launch_count = 0;
    const int rc = run_step(false);
    if (rc != ORION_OK) {
      only_mask_ = 0;
      return rc;
    }
    last_launches_ = g_launch_count;
  }
  only_mask_ = 0;
  ORION_CUDA_CHECK("replay", cudaEventRecord(ev1_, stream_));
  ORION_TRY(wait_for(stream_, "replay"));
  ORION_CUDA_CHECK("replay", cudaEventSynchronize(ev1_));
  float ms = 0.f;
  ORION_CUDA_CHECK("replay", cudaEventElapsedTime(&ms, ev0_, ev1_));
  if (elapsed_ms) *elapsed_ms = ms;
  return ORION_OK;
}

template <typename T>
int Model<T>::profile(int iterations, float category_ms[kProfCategories],
                      uint64_t category_launches[kProfCategories]) {
  if (meta_.rows == 0 || meta_.zero_count)
    return set_error(ORION_ERR_INVALID_REQUEST, "profile needs a preceding successful forward");
  ORION_CUDA_CHECK("set device", cudaSetDevice(ordinal_));
  for (int c = 0; c < kProfCategories; ++c) {
    category_ms[c] = 0.f;
    category_launches[c] = 0;
  }
  for (int i = 0; i < iterations; ++i) {
    prof_recs_.clear();
    prof_used_ = 0;
    prof_on_ = true;
    const int rc = run_step(false);
    prof_on_ = false;
    ORION_TRY(rc);
    ORION_CUDA_CHECK("profile", cudaStreamSynchronize(stream_));
    for (const ProfRec &r : prof_recs_) {
      float ms = 0.f;
      ORION_CUDA_CHECK("profile", cudaEventElapsedTime(&ms, r.a, r.b));
      category_ms[r.cat] += ms;
      category_launches[r.cat] += 1;
    }
  }
  return ORION_OK;
}

template <typename T>
int Model<T>::fill_kv_random(uint64_t seed, float std) {
  ORION_CUDA_CHECK("set device", cudaSetDevice(ordinal_));
  const size_t total = kv_.layer_elems() * d_.num_layers;
  const size_t chunk = 64u << 20;
  ORION_TRY(ensure_stage(&stage_f32_, &stage_f32_cap_, std::min(total, chunk) * sizeof(float)));
  for (size_t off = 0; off < total; off += chunk) {
    const size_t m = std::min(chunk, total - off);
    float *tmp = static_cast<float *>(stage_f32_);
    ORION_TRY(launch_fill_normal<float>(tmp, m, seed + off, stream_));
    ORION_TRY(launch_scale_convert<T>(tmp, arena_ + off, m, std, stream_));
  }
  ORION_CUDA_CHECK("fill_kv_random", cudaStreamSynchronize(stream_));
  return ORION_OK;
}

template <typename T>
int Model<T>::read_kv(float *out, uint64_t capacity) {
  const size_t total = kv_.layer_elems() * d_.num_layers;
  if (capacity < total)
    return set_error(ORION_ERR_INVALID_REQUEST, "KV read-back buffer holds %llu floats, %zu needed",
                     (unsigned long long)capacity, total);
  ORION_CUDA_CHECK("set device", cudaSetDevice(ordinal_));
  float *tmp = nullptr;
  ORION_CUDA_CHECK("allocate", cudaMalloc(&tmp, (total ? total : 1) * sizeof(float)));
  int rc = launch_arena_to_reference_order<T>(arena_, kv_, tmp, stream_);
  if (rc == ORION_OK) {
    cudaError_t e = cudaMemcpyAsync(out, tmp, total * sizeof(float), cudaMemcpyDeviceToHost, stream_);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream_);
    if (e != cudaSuccess) rc = set_error(ORION_ERR_BACKEND, "backend cuda failed at read_kv: %s", cudaGetErrorString(e));
  }
  cudaFree(tmp);
  return rc;
}

}  // namespace

int create_model(OrionBackend *backend, const OrionModelDesc *desc, ModelBase **out) {
  *out = nullptr;
  if (desc->compute_dtype == ORION_DTYPE_F32) {
    auto *m = new Model<float>(backend, *desc);
    int rc = m->init();
    if (rc != ORION_OK) { delete m; return rc; }
    *out = m;
    return ORION_OK;
  }
  if (desc->compute_dtype == ORION_DTYPE_BF16) {
    auto *m = new Model<bf16>(backend, *desc);
    int rc = m->init();
    if (rc != ORION_OK) { delete m; return rc; }
    *out = m;
    return ORION_OK;
  }
  return set_error(ORION_ERR_MODEL, "unsupported compute dtype %u (f32 and bf16 are implemented)", desc->compute_dtype);
}

}  // namespace orion
