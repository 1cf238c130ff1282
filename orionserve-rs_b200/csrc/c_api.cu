// extern "C" entry points declared in include/orion_cuda.h.
#include <cstring>
#include <memory>
#include <new>
#include <vector>

#include "model.h"

namespace orion {

namespace {
thread_local char g_error[1024] = "";
}

int set_error(int status, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return status;
}
void clear_error() { g_error[0] = '\0'; }

namespace {

// RAII device buffer for the op-level entry points.
template <typename U>
struct Dev {
  U *p = nullptr;
  ~Dev() { if (p) cudaFree(p); }
  int alloc(size_t n) {
    ORION_CUDA_CHECK("allocate", cudaMalloc(reinterpret_cast<void **>(&p), (n ? n : 1) * sizeof(U)));
    return ORION_OK;
  }
  int upload(const U *h, size_t n) {
    ORION_TRY(alloc(n));
    if (n) ORION_CUDA_CHECK("upload", cudaMemcpy(p, h, n * sizeof(U), cudaMemcpyHostToDevice));
    return ORION_OK;
  }
};

template <typename T>
int to_storage(const float *host, size_t n, Dev<float> *f32, Dev<T> *out) {
  ORION_TRY(f32->upload(host, n));
  ORION_TRY(out->alloc(n));
  return launch_convert_from_f32<T>(f32->p, out->p, n, 0);
}

int check_backend(const OrionBackend *b) {
  if (!b) return set_error(ORION_ERR_INVALID_REQUEST, "null backend handle");
  ORION_CUDA_CHECK("set device", cudaSetDevice(b->ordinal));
  return ORION_OK;
}

int rope_tables(uint64_t head_dim, uint64_t max_positions, float theta, Dev<float> *c, Dev<float> *s) {
  if (head_dim % 2 != 0)  // tensor.rs:229-233
    return set_error(ORION_ERR_INTERNAL, "RoPE requires an even head_dim, got %llu", (unsigned long long)head_dim);
  const size_t half = head_dim / 2, n = max_positions * half;
  std::vector<float> hc(n ? n : 1), hs(n ? n : 1);
  for (size_t pos = 0; pos < max_positions; ++pos)
    for (size_t i = 0; i < half; ++i) {  // tensor.rs:238-246
      const float inv_freq = 1.0f / powf(theta, 2.0f * (float)i / (float)head_dim);
      const float angle = (float)pos * inv_freq;
      hc[pos * half + i] = cosf(angle);
      hs[pos * half + i] = sinf(angle);
    }
  ORION_TRY(c->upload(hc.data(), n));
  return s->upload(hs.data(), n);
}

template <typename T>
int op_linear(const float *x, uint64_t rows, uint64_t k, const float *w, uint64_t n, const float *bias, float *out) {
  Dev<float> xf, wf, bf_, part, res;
  Dev<T> xt, wt;
  ORION_TRY(to_storage<T>(x, rows * k, &xf, &xt));
  ORION_TRY(to_storage<T>(w, n * k, &wf, &wt));
  if (bias) ORION_TRY(bf_.upload(bias, n));
  constexpr bool kBf16 = sizeof(T) == 2;
  GemmPlan p = gemm_plan(kBf16, (uint32_t)rows, (uint32_t)n, (uint32_t)k, (uint32_t)k, (uint32_t)k);
  ORION_TRY(part.alloc((size_t)p.splits * rows * n));
  ORION_TRY(res.alloc(rows * n));
  ORION_TRY(launch_gemm<T>(xt.p, (uint32_t)k, wt.p, (uint32_t)k, part.p, (uint32_t)rows, (uint32_t)n, (uint32_t)k, p, 0));
  ORION_TRY(launch_finish_linear(part.p, p.out_slabs, rows * n, bias ? bf_.p : nullptr, res.p, (uint32_t)rows, (uint32_t)n, 0));
  ORION_CUDA_CHECK("linear", cudaMemcpy(out, res.p, rows * n * sizeof(float), cudaMemcpyDeviceToHost));
  uint32_t code = 0;
  if (kBf16) {
    ORION_TRY(gemm_tc_poll_error(&code));
    if (code) return set_error(ORION_ERR_BACKEND, "backend cuda failed at gemm: a bounded pipeline wait ran out (code %u)", code);
  }
  return ORION_OK;
}

template <typename T>
int op_rms_norm(float *x, uint64_t rows, uint64_t cols, const float *w, float eps) {
  Dev<float> xf, wf, back;
  Dev<T> o;
  ORION_TRY(xf.upload(x, rows * cols));
  ORION_TRY(wf.upload(w, cols));
  ORION_TRY(o.alloc(rows * cols));
  ORION_TRY(back.alloc(rows * cols));
  if (sizeof(T) == 2) {  // bf16 kernels see bf16-rounded activations
    Dev<T> xr;
    ORION_TRY(xr.alloc(rows * cols));
    ORION_TRY(launch_convert_from_f32<T>(xf.p, xr.p, rows * cols, 0));
    ORION_TRY(launch_convert_to_f32<T>(xr.p, xf.p, rows * cols, 0));
    ORION_CUDA_CHECK("rms_norm", cudaDeviceSynchronize());
  }
  ORION_TRY(launch_rmsnorm_rows<T>(xf.p, wf.p, eps, o.p, (uint32_t)rows, (uint32_t)cols, 0));
  ORION_TRY(launch_convert_to_f32<T>(o.p, back.p, rows * cols, 0));
  ORION_CUDA_CHECK("rms_norm", cudaMemcpy(x, back.p, rows * cols * sizeof(float), cudaMemcpyDeviceToHost));
  return ORION_OK;
}

template <typename T>
int op_swiglu(float *gate, const float *up, uint64_t rows, uint64_t cols) {
  // The kernel reads [rows][2*cols] (gate | up), the layout of the fused projection.
  std::vector<float> gu(rows * cols * 2);
  for (uint64_t r = 0; r < rows; ++r) {
    std::memcpy(&gu[r * 2 * cols], gate + r * cols, cols * sizeof(float));
    std::memcpy(&gu[r * 2 * cols + cols], up + r * cols, cols * sizeof(float));
  }
  Dev<float> in, back;
  Dev<T> act;
  ORION_TRY(in.upload(gu.data(), gu.size()));
  ORION_TRY(act.alloc(rows * cols));
  ORION_TRY(back.alloc(rows * cols));
  ORION_TRY(launch_swiglu<T>(in.p, 1, 0, act.p, (uint32_t)rows, (uint32_t)cols, 0));
  ORION_TRY(launch_convert_to_f32<T>(act.p, back.p, rows * cols, 0));
  ORION_CUDA_CHECK("swiglu", cudaMemcpy(gate, back.p, rows * cols * sizeof(float), cudaMemcpyDeviceToHost));
  return ORION_OK;
}

template <typename T>
int op_rope(float *x, uint64_t rows, uint64_t heads, uint64_t hd, const uint32_t *positions, uint64_t max_pos, float theta) {
  Dev<float> c, s, xf, back;
  Dev<T> xt;
  Dev<uint32_t> pos;
  ORION_TRY(rope_tables(hd, max_pos, theta, &c, &s));
  for (uint64_t r = 0; r < rows; ++r)  // transformer.rs:257-262
    if (positions[r] >= max_pos)
      return set_error(ORION_ERR_INTERNAL, "position %u exceeds the RoPE table (%llu entries)", positions[r],
                       (unsigned long long)max_pos);
  const size_t n = rows * heads * hd;
  ORION_TRY(to_storage<T>(x, n, &xf, &xt));
  ORION_TRY(pos.upload(positions, rows));
  ORION_TRY(back.alloc(n));
  ORION_TRY(launch_rope_rows<T>(xt.p, pos.p, c.p, s.p, (uint32_t)rows, (uint32_t)heads, (uint32_t)hd, 0));
  ORION_TRY(launch_convert_to_f32<T>(xt.p, back.p, n, 0));
  ORION_CUDA_CHECK("rope", cudaMemcpy(x, back.p, n * sizeof(float), cudaMemcpyDeviceToHost));
  return ORION_OK;
}

template <typename T>
int op_attention(const float *kv, uint64_t num_blocks, uint64_t block_size, uint64_t kvh, uint64_t hd,
                 const float *query, uint64_t rows, uint64_t qh, const uint32_t *qpos,
                 const uint32_t *seq_of_row, const uint32_t *tables, const uint64_t *offsets,
                 uint64_t nseq, float *out) {
  KvLayout lay{1, (uint32_t)num_blocks, (uint32_t)kvh, (uint32_t)block_size, (uint32_t)hd,
               (sizeof(T) == 2 && hd % 64 == 0) ? 1u : 0u};
  const size_t arena_n = lay.layer_elems();
  Dev<float> ref, qf, back;
  Dev<T> arena, qt, ot;
  Dev<uint32_t> dpos, dseq, dtab, doff;
  ORION_TRY(ref.upload(kv, arena_n));
  ORION_TRY(arena.alloc(arena_n));
  ORION_TRY(launch_arena_from_reference_order<T>(ref.p, lay, arena.p, 0));
  const size_t qn = rows * qh * hd;
  ORION_TRY(to_storage<T>(query, qn, &qf, &qt));
  ORION_TRY(ot.alloc(qn));
  ORION_TRY(back.alloc(qn));
  std::vector<uint32_t> off32(nseq + 1);
  for (uint64_t i = 0; i <= nseq; ++i) off32[i] = (uint32_t)offsets[i];
  uint32_t max_pos = 0;
  bool decode = rows == nseq;
  for (uint64_t r = 0; r < rows; ++r) {
    max_pos = std::max(max_pos, qpos[r]);
    decode = decode && seq_of_row[r] == r;
  }
  ORION_TRY(dpos.upload(qpos, rows));
  ORION_TRY(dseq.upload(seq_of_row, rows));
  ORION_TRY(dtab.upload(tables, offsets[nseq]));
  ORION_TRY(doff.upload(off32.data(), nseq + 1));
  AttnBatch ab{dpos.p, dseq.p, dtab.p, doff.p, (uint32_t)rows, max_pos};
  bool done = false;
  if constexpr (sizeof(T) == 2) {
    if (decode && decode_attention_supported(lay, (uint32_t)qh)) {
      uint64_t total_blocks = 0;
      for (uint64_t r = 0; r < rows; ++r) total_blocks += qpos[r] / block_size + 1;
      const DecodePlan plan = decode_plan((uint32_t)rows, (uint32_t)kvh, total_blocks, max_pos, (uint32_t)block_size, 32);
      const uint32_t splits = plan.splits;
      Dev<float> scratch;
      const size_t scratch_floats = decode_scratch_floats((uint32_t)rows, (uint32_t)qh, (uint32_t)hd, splits);
      ORION_TRY(scratch.alloc(scratch_floats));
      ORION_CUDA_CHECK("clear attention scratch", cudaMemset(scratch.p, 0, scratch_floats * sizeof(float)));
      DecodeScratch sc = decode_scratch_at(scratch.p, (uint32_t)rows, (uint32_t)qh, (uint32_t)kvh, (uint32_t)hd, splits,
                                           plan.blocks_per_split);
      ORION_TRY(launch_paged_attention_decode(qt.p, arena.p, lay, 0, ab, (uint32_t)qh, splits, sc, ot.p, 0));
      ORION_CUDA_CHECK("paged_attention", cudaDeviceSynchronize());
      uint32_t code = 0;
      ORION_TRY(decode_poll_error(&code));
      if (code) return set_error(ORION_ERR_BACKEND, "backend cuda failed at attention: a bounded pipeline wait ran out (code %u)", code);
      done = true;
    }
  }
  if constexpr (sizeof(T) == 2) {
    if (!done && prefill_attention_supported(lay, (uint32_t)qh)) {
      // tiles of consecutive rows of one sequence, like the model builds them
      const uint32_t tile_rows = prefill_tile_positions((uint32_t)qh, (uint32_t)kvh);
      std::vector<PrefillTile> tiles;
      for (uint64_t r = 0; r < rows;) {
        PrefillTile t{(uint32_t)r, 0, seq_of_row[r], 0};
        while (r < rows && seq_of_row[r] == t.seq && t.num_rows < tile_rows) {
          t.max_position = std::max(t.max_position, qpos[r]);
          ++t.num_rows;
          ++r;
        }
        tiles.push_back(t);
      }
      Dev<PrefillTile> dt;
      ORION_TRY(dt.upload(tiles.data(), tiles.size()));
      ORION_TRY(launch_paged_attention_prefill(qt.p, arena.p, lay, 0, ab, dt.p, (uint32_t)tiles.size(), (uint32_t)qh, ot.p, 0));
      ORION_CUDA_CHECK("paged_attention", cudaDeviceSynchronize());
      uint32_t code = 0;
      ORION_TRY(prefill_poll_error(&code));
      if (code) return set_error(ORION_ERR_BACKEND, "backend cuda failed at prefill attention: a bounded pipeline wait ran out (code %u)", code);
      done = true;
    }
  }
  if (!done) ORION_TRY(launch_paged_attention_generic<T>(qt.p, arena.p, lay, 0, ab, (uint32_t)qh, ot.p, 0));
  ORION_TRY(launch_convert_to_f32<T>(ot.p, back.p, qn, 0));
  ORION_CUDA_CHECK("paged_attention", cudaMemcpy(out, back.p, qn * sizeof(float), cudaMemcpyDeviceToHost));
  return ORION_OK;
}

int bad_dtype(int dtype) {
  return set_error(ORION_ERR_INVALID_REQUEST, "dtype %d is not executable on this backend (f32 and bf16 are)", dtype);
}

}  // namespace
}  // namespace orion

using namespace orion;

struct OrionAttnBench {
  OrionBackend *backend = nullptr;
  KvLayout lay{};
  uint32_t q_heads = 0, batch = 0, splits = 1, blocks_per_split = 0, max_position = 0;
  bf16 *arena = nullptr, *q = nullptr, *out = nullptr;
  uint32_t *meta = nullptr;  // positions | seq_of_row | offsets | tables
  float *scratch = nullptr;
  std::vector<uint32_t> ctx, offsets, tables;
  uint64_t algorithmic_bytes = 0;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  ~OrionAttnBench() {
    cudaFree(arena); cudaFree(q); cudaFree(out); cudaFree(meta); cudaFree(scratch);
    if (ev0) cudaEventDestroy(ev0);
    if (ev1) cudaEventDestroy(ev1);
  }
};

// ---- Collective over NCCL (orion-distributed/src/lib.rs:231-254), host buffers in and out ----

struct OrionCollective {
  int ordinal = 0;
  cudaStream_t stream = nullptr;
  orion::NcclCollective nccl;
  float *dev = nullptr;
  size_t cap = 0;
  ~OrionCollective() {
    cudaSetDevice(ordinal);
    if (dev) cudaFree(dev);
    if (stream) cudaStreamDestroy(stream);
  }
  int reserve(size_t floats) {
    if (cap >= floats) return ORION_OK;
    if (dev) cudaFree(dev);
    dev = nullptr;
    cap = 0;
    ORION_CUDA_CHECK("allocate", cudaMalloc(reinterpret_cast<void **>(&dev), (floats ? floats : 1) * sizeof(float)));
    cap = floats;
    return ORION_OK;
  }
};

namespace {
// in: `in_count` floats from the host; the collective; out: `out_count` floats back to the host.
template <typename F>
int collective_round_trip(OrionCollective *c, const float *in, size_t in_count, float *out, size_t out_count,
                          const char *stage, F &&run) {
  orion::clear_error();
  if (!c || (in_count && !in) || (out_count && !out)) return orion::set_error(ORION_ERR_INVALID_REQUEST, "null argument");
  ORION_CUDA_CHECK("set device", cudaSetDevice(c->ordinal));
  ORION_TRY(c->reserve(in_count + out_count));
  float *d_in = c->dev, *d_out = c->dev + in_count;
  if (in_count)
    ORION_CUDA_CHECK(stage, cudaMemcpyAsync(d_in, in, in_count * sizeof(float), cudaMemcpyHostToDevice, c->stream));
  ORION_TRY(run(d_in, d_out));
  if (out_count)
    ORION_CUDA_CHECK(stage, cudaMemcpyAsync(out, d_out, out_count * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  return c->nccl.wait_stream(c->stream, stage);
}
}  // namespace

extern "C" {

const char *orion_cuda_last_error(void) { return g_error; }

int orion_cuda_is_available(void) { return orion_cuda_device_count() > 0; }

int orion_cuda_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int orion_cuda_backend_create(int ordinal, OrionBackend **out) {
  clear_error();
  if (!out) return set_error(ORION_ERR_INVALID_REQUEST, "null output pointer");
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver || e != cudaSuccess) {
    cudaGetLastError();
    if (e == cudaErrorInsufficientDriver || e == cudaErrorInitializationError)
      return set_error(ORION_ERR_UNAVAILABLE, "no CUDA driver found");  // CudaUnavailable::NoDriver
    return set_error(ORION_ERR_UNAVAILABLE, "CUDA driver found but no devices available");
  }
  if (n == 0) return set_error(ORION_ERR_UNAVAILABLE, "CUDA driver found but no devices available");
  if (ordinal < 0 || ordinal >= n)  // CudaUnavailable::NoSuchDevice
    return set_error(ORION_ERR_UNAVAILABLE, "CUDA device %d requested but only %d device(s) present", ordinal, n);
  cudaDeviceProp prop;
  ORION_CUDA_CHECK("device properties", cudaGetDeviceProperties(&prop, ordinal));
  if (prop.major != 10)
    return set_error(ORION_ERR_UNAVAILABLE, "CUDA device %d is sm_%d%d; this library is built for sm_100a only",
                     ordinal, prop.major, prop.minor);
  ORION_CUDA_CHECK("set device", cudaSetDevice(ordinal));
  auto *b = new (std::nothrow) OrionBackend();
  if (!b) return set_error(ORION_ERR_INTERNAL, "out of host memory");
  b->ordinal = ordinal;
  b->device_name = prop.name;
  b->total_memory = prop.totalGlobalMem;
  *out = b;
  return ORION_OK;
}

void orion_cuda_backend_destroy(OrionBackend *backend) { delete backend; }
const char *orion_cuda_backend_name(const OrionBackend *) { return "cuda"; }
int orion_cuda_backend_ordinal(const OrionBackend *backend) { return backend ? backend->ordinal : -1; }
const char *orion_cuda_backend_device_name(const OrionBackend *backend) {
  return backend ? backend->device_name.c_str() : "";
}

int orion_cuda_backend_total_memory(const OrionBackend *backend, uint64_t *bytes) {
  clear_error();
  ORION_TRY(check_backend(backend));
  *bytes = backend->total_memory;
  return ORION_OK;
}

int orion_cuda_backend_available_memory(const OrionBackend *backend, uint64_t *bytes) {
  clear_error();
  ORION_TRY(check_backend(backend));
  size_t free_b = 0, total_b = 0;
  ORION_CUDA_CHECK("available_memory", cudaMemGetInfo(&free_b, &total_b));
  *bytes = free_b;
  return ORION_OK;
}

int orion_cuda_backend_synchronize(const OrionBackend *backend) {
  clear_error();
  ORION_TRY(check_backend(backend));
  ORION_CUDA_CHECK("synchronize", cudaDeviceSynchronize());
  return ORION_OK;
}

int orion_cuda_backend_supports_dtype(const OrionBackend *, int dtype) {
  return dtype == ORION_DTYPE_F32 || dtype == ORION_DTYPE_BF16;
}

int orion_cuda_model_create(OrionBackend *backend, const OrionModelDesc *desc, OrionModel **out) {
  clear_error();
  if (!out || !desc) return set_error(ORION_ERR_INVALID_REQUEST, "null pointer argument");
  *out = nullptr;
  ORION_TRY(check_backend(backend));
  ModelBase *impl = nullptr;
  ORION_TRY(create_model(backend, desc, &impl));
  auto *m = new (std::nothrow) OrionModel();
  if (!m) { delete impl; return set_error(ORION_ERR_INTERNAL, "out of host memory"); }
  m->impl.reset(impl);
  *out = m;
  return ORION_OK;
}

void orion_cuda_model_destroy(OrionModel *model) { delete model; }

int orion_cuda_model_load_tensor(OrionModel *model, const char *name, int dtype, const uint64_t *shape, int ndim,
                                 const void *data) {
  clear_error();
  if (!model || !name || !shape) return set_error(ORION_ERR_INVALID_REQUEST, "null pointer argument");
  return model->impl->load_tensor(name, dtype, shape, ndim, data);
}

int orion_cuda_model_init_random(OrionModel *model, uint64_t seed, float std) {
  clear_error();
  if (!model) return set_error(ORION_ERR_INVALID_REQUEST, "null model handle");
  return model->impl->init_random(seed, std);
}

int orion_cuda_model_finalize(OrionModel *model) {
  clear_error();
  if (!model) return set_error(ORION_ERR_INVALID_REQUEST, "null model handle");
  return model->impl->finalize();
}

int orion_cuda_model_forward_greedy(OrionModel *model, const uint32_t *tokens, uint64_t num_tokens,
                                    const uint32_t *positions, uint64_t num_positions,
                                    const uint64_t *slot_token_counts, uint64_t num_slot_token_counts,
                                    const uint64_t *context_lens, uint64_t num_context_lens,
                                    const uint32_t *block_tables_flat, const uint64_t *block_table_offsets,
                                    uint64_t num_block_tables, uint64_t num_sequences, int has_prefill,
                                    uint32_t *token_ids_out, float *logits_out, uint64_t logits_capacity) {
  clear_error();
  if (!model) return set_error(ORION_ERR_INVALID_REQUEST, "null model handle");
  BatchView b{tokens, num_tokens, positions, num_positions, slot_token_counts, num_slot_token_counts,
              context_lens, num_context_lens, block_tables_flat, block_table_offsets, num_block_tables,
              num_sequences, has_prefill};
  return model->impl->forward(b, logits_out, logits_capacity, token_ids_out);
}

int orion_cuda_model_forward(OrionModel *model, const uint32_t *tokens, uint64_t num_tokens,
                             const uint32_t *positions, uint64_t num_positions,
                             const uint64_t *slot_token_counts, uint64_t num_slot_token_counts,
                             const uint64_t *context_lens, uint64_t num_context_lens,
                             const uint32_t *block_tables_flat, const uint64_t *block_table_offsets,
                             uint64_t num_block_tables, uint64_t num_sequences, int has_prefill,
                             float *logits_out, uint64_t logits_capacity) {
  return orion_cuda_model_forward_greedy(model, tokens, num_tokens, positions, num_positions, slot_token_counts,
                                         num_slot_token_counts, context_lens, num_context_lens, block_tables_flat,
                                         block_table_offsets, num_block_tables, num_sequences, has_prefill, nullptr,
                                         logits_out, logits_capacity);
}

int orion_cuda_selftest_bounded_wait(OrionBackend *backend, uint64_t limit_us, uint32_t *timed_out, uint32_t *waited_us) {
  clear_error();
  ORION_TRY(check_backend(backend));
  return selftest_bounded_wait(limit_us, timed_out, waited_us);
}

int orion_cuda_collective_create(OrionBackend *backend, const uint8_t id[ORION_NCCL_ID_BYTES], uint32_t rank,
                                 uint32_t world, OrionCollective **out) {
  orion::clear_error();
  ORION_TRY(orion::check_backend(backend));
  if (!id || !out) return orion::set_error(ORION_ERR_INVALID_REQUEST, "null argument");
  *out = nullptr;
  if (world == 0) return orion::set_error(ORION_ERR_INVALID_REQUEST, "world_size must be at least 1");  // Rank::new
  if (rank >= world)
    return orion::set_error(ORION_ERR_INVALID_REQUEST, "rank %u is out of range for world size %u", rank, world);
  std::unique_ptr<OrionCollective> c(new (std::nothrow) OrionCollective());
  if (!c) return orion::set_error(ORION_ERR_INTERNAL, "out of host memory");
  c->ordinal = backend->ordinal;
  ORION_CUDA_CHECK("create stream", cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
  if (world > 1) ORION_TRY(c->nccl.init(id, (int)rank, (int)world));
  *out = c.release();
  return ORION_OK;
}

void orion_cuda_collective_destroy(OrionCollective *c) { delete c; }

int orion_cuda_collective_all_reduce_sum(OrionCollective *c, float *buffer, uint64_t count) {
  return collective_round_trip(c, buffer, count, nullptr, 0, "all_reduce_sum", [&](float *d_in, float *) -> int {
    ORION_TRY(c->nccl.all_reduce_sum(d_in, count, c->stream));
    if (count)  // in place: the sum goes back into the caller's buffer
      ORION_CUDA_CHECK("all_reduce_sum", cudaMemcpyAsync(buffer, d_in, count * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
    return ORION_OK;
  });
}

int orion_cuda_collective_all_gather(OrionCollective *c, const float *local, uint64_t count_per_rank, float *out) {
  const size_t world = c ? (size_t)c->nccl.world() : 1;
  return collective_round_trip(c, local, count_per_rank, out, count_per_rank * world, "all_gather",
                               [&](float *d_in, float *d_out) { return c->nccl.all_gather(d_in, d_out, count_per_rank, c->stream); });
}

int orion_cuda_collective_reduce_scatter_sum(OrionCollective *c, const float *input, uint64_t count_per_rank, float *out) {
  const size_t world = c ? (size_t)c->nccl.world() : 1;
  return collective_round_trip(c, input, count_per_rank * world, out, count_per_rank, "reduce_scatter_sum",
                               [&](float *d_in, float *d_out) { return c->nccl.reduce_scatter_sum(d_in, d_out, count_per_rank, c->stream); });
}

int orion_cuda_collective_barrier(OrionCollective *c) {
  orion::clear_error();
  if (!c) return orion::set_error(ORION_ERR_INVALID_REQUEST, "null argument");
  ORION_CUDA_CHECK("set device", cudaSetDevice(c->ordinal));
  return c->nccl.barrier(c->stream);
}

int orion_cuda_selftest_peer_wait(OrionBackend *backend, uint64_t limit_us, uint32_t *timed_out, uint32_t *waited_us) {
  orion::clear_error();
  ORION_TRY(orion::check_backend(backend));
  return orion::selftest_peer_wait(limit_us, timed_out, waited_us);
}

int orion_cuda_tp_selftest_failure_handling(int scenario, uint64_t limit_ms, uint32_t *aborted, uint64_t *polls) {
  orion::clear_error();
  return orion::nccl_failure_selftest(scenario, limit_ms, aborted, polls);
}

int orion_cuda_poll_wait_timeouts(OrionBackend *backend, uint32_t *mask) {
  orion::clear_error();
  ORION_TRY(orion::check_backend(backend));
  if (!mask) return orion::set_error(ORION_ERR_INVALID_REQUEST, "null output pointer");
  uint32_t gemm = 0, decode = 0, prefill = 0, tp = 0;
  ORION_TRY(orion::gemm_tc_poll_error(&gemm));
  ORION_TRY(orion::decode_poll_error(&decode));
  ORION_TRY(orion::prefill_poll_error(&prefill));
  ORION_TRY(orion::tp_poll_error(&tp));
  *mask = (gemm ? 1u : 0u) | (decode ? 2u : 0u) | (prefill ? 4u : 0u) | (tp ? 8u : 0u);
  return ORION_OK;
}

int orion_cuda_model_load_checkpoint(OrionModel *model, const char *directory, uint64_t *tensors_loaded) {
  clear_error();
  if (!model) return set_error(ORION_ERR_INVALID_REQUEST, "null model handle");
  return load_checkpoint(model->impl.get(), directory, tensors_loaded);
}

int orion_cuda_model_replay(OrionModel *model, int iterations, float *elapsed_ms) {
  clear_error();
  if (!model) return set_error(ORION_ERR_INVALID_REQUEST, "null model handle");
  return model->impl->replay(iterations, 0, elapsed_ms);
}

int orion_cuda_model_replay_categories(OrionModel *model, int iterations, uint32_t category_mask, float *elapsed_ms) {
  clear_error();
  if (!model) return set_error(ORION_ERR_INVALID_REQUEST, "null model handle");
  if (category_mask == 0 || category_mask >= (1u << kProfCategories))
    return set_error(ORION_ERR_INVALID_REQUEST, "category mask must name at least one of the four kernel categories");
  return model->impl->replay(iterations, category_mask, elapsed_ms);
}

int orion_cuda_model_profile(OrionModel *model, int iterations, float category_ms[4],
                             uint64_t category_launches[4]) {
  clear_error();
  if (!model || !category_ms || !category_launches)
    return set_error(ORION_ERR_INVALID_REQUEST, "null pointer argument");
  return model->impl->profile(iterations, category_ms, category_launches);
}

int orion_cuda_model_fill_kv_random(OrionModel *model, uint64_t seed, float std) {
  clear_error();
  if (!model) return set_error(ORION_ERR_INVALID_REQUEST, "null model handle");
  return model->impl->fill_kv_random(seed, std);
}

int orion_cuda_model_last_launch_count(const OrionModel *model, uint64_t *launches) {
  clear_error();
  if (!model || !launches) return set_error(ORION_ERR_INVALID_REQUEST, "null pointer argument");
  *launches = model->impl->last_launch_count();
  return ORION_OK;
}

int orion_cuda_model_read_kv(OrionModel *model, float *out, uint64_t capacity) {
  clear_error();
  if (!model || !out) return set_error(ORION_ERR_INVALID_REQUEST, "null pointer argument");
  return model->impl->read_kv(out, capacity);
}

int orion_cuda_model_desc(const OrionModel *model, OrionModelDesc *out) {
  clear_error();
  if (!model || !out) return set_error(ORION_ERR_INVALID_REQUEST, "null pointer argument");
  *out = model->impl->desc();
  return ORION_OK;
}

int orion_cuda_tp_layout(uint32_t num_attention_heads, uint32_t num_kv_heads, uint32_t ffn_dim, uint32_t rank,
                         uint32_t world, uint64_t query_heads[2], uint64_t kv_heads[2], uint64_t ffn[2]) {
  clear_error();
  ParallelLayout l;
  ORION_TRY(compute_layout(num_attention_heads, num_kv_heads, ffn_dim, rank, world, &l));
  query_heads[0] = l.query_heads.start; query_heads[1] = l.query_heads.len;
  kv_heads[0] = l.kv_heads.start; kv_heads[1] = l.kv_heads.len;
  ffn[0] = l.ffn.start; ffn[1] = l.ffn.len;
  return ORION_OK;
}

int orion_cuda_tp_unique_id(uint8_t id[ORION_NCCL_ID_BYTES]) {
  clear_error();
  return NcclCollective::unique_id(id);
}

void *orion_cuda_host_alloc(uint64_t bytes) {
  void *p = nullptr;
  if (cudaMallocHost(&p, bytes ? bytes : 1) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}
void orion_cuda_host_free(void *p) { if (p) cudaFreeHost(p); }

int orion_cuda_set_programmatic_launch(int enabled) {
  g_pdl_enabled = enabled != 0;
  ++g_tuning_generation;
  return ORION_OK;
}

int orion_cuda_attention_set_tuning(int stages, uint32_t cta_target) {
  decode_set_tuning(stages, cta_target);
  ++g_tuning_generation;
  return ORION_OK;
}

int orion_cuda_gemm_set_tuning(uint32_t ctas, int small_batch_stages) {
  if (small_batch_stages) gemm_set_small_stages(small_batch_stages);
  gemm_set_target_ctas(ctas);
  ++g_tuning_generation;
  return ORION_OK;
}

// ---- op-level entry points -------------------------------------------------------

int orion_cuda_linear(OrionBackend *backend, int dtype, const float *x, uint64_t rows, uint64_t in_features,
                      const float *weight, uint64_t out_features, uint64_t weight_in_features, const float *bias,
                      uint64_t bias_len, float *out) {
  clear_error();
  ORION_TRY(check_backend(backend));
  if (in_features != weight_in_features)  // tensor.rs:100-104
    return set_error(ORION_ERR_INTERNAL, "linear shape mismatch: input has %llu features, weight expects %llu",
                     (unsigned long long)in_features, (unsigned long long)weight_in_features);
  if (bias && bias_len != out_features)  // tensor.rs:105-112
    return set_error(ORION_ERR_INTERNAL, "bias has %llu elements, expected %llu", (unsigned long long)bias_len,
                     (unsigned long long)out_features);
  if (rows == 0 || out_features == 0) return ORION_OK;
  if (dtype == ORION_DTYPE_F32) return op_linear<float>(x, rows, in_features, weight, out_features, bias, out);
  if (dtype == ORION_DTYPE_BF16) return op_linear<bf16>(x, rows, in_features, weight, out_features, bias, out);
  return bad_dtype(dtype);
}

int orion_cuda_rms_norm(OrionBackend *backend, int dtype, float *x, uint64_t rows, uint64_t cols, const float *weight,
                        uint64_t weight_len, float eps) {
  clear_error();
  ORION_TRY(check_backend(backend));
  if (weight_len != cols)  // tensor.rs:145-150
    return set_error(ORION_ERR_INTERNAL, "rms_norm weight has %llu elements, expected %llu",
                     (unsigned long long)weight_len, (unsigned long long)cols);
  if (rows == 0 || cols == 0) return ORION_OK;
  if (dtype == ORION_DTYPE_F32) return op_rms_norm<float>(x, rows, cols, weight, eps);
  if (dtype == ORION_DTYPE_BF16) return op_rms_norm<bf16>(x, rows, cols, weight, eps);
  return bad_dtype(dtype);
}

int orion_cuda_swiglu(OrionBackend *backend, int dtype, float *gate, uint64_t gate_rows, uint64_t gate_cols,
                      const float *up, uint64_t up_rows, uint64_t up_cols) {
  clear_error();
  ORION_TRY(check_backend(backend));
  if (gate_rows != up_rows || gate_cols != up_cols)  // tensor.rs:176-184
    return set_error(ORION_ERR_INTERNAL, "swiglu shape mismatch: gate is %llux%llu, up is %llux%llu",
                     (unsigned long long)gate_rows, (unsigned long long)gate_cols, (unsigned long long)up_rows,
                     (unsigned long long)up_cols);
  if (gate_rows == 0 || gate_cols == 0) return ORION_OK;
  if (dtype == ORION_DTYPE_F32) return op_swiglu<float>(gate, up, gate_rows, gate_cols);
  if (dtype == ORION_DTYPE_BF16) return op_swiglu<bf16>(gate, up, gate_rows, gate_cols);
  return bad_dtype(dtype);
}

int orion_cuda_rope(OrionBackend *backend, int dtype, float *x, uint64_t rows, uint64_t heads, uint64_t head_dim,
                    const uint32_t *positions, uint64_t max_positions, float theta) {
  clear_error();
  ORION_TRY(check_backend(backend));
  if (rows == 0 || heads == 0) return ORION_OK;
  if (dtype == ORION_DTYPE_F32) return op_rope<float>(x, rows, heads, head_dim, positions, max_positions, theta);
  if (dtype == ORION_DTYPE_BF16) return op_rope<bf16>(x, rows, heads, head_dim, positions, max_positions, theta);
  return bad_dtype(dtype);
}

int orion_cuda_paged_attention(OrionBackend *backend, int dtype, const float *kv, uint64_t num_blocks,
                               uint64_t block_size, uint64_t num_kv_heads, uint64_t head_dim, const float *query,
                               uint64_t rows, uint64_t num_query_heads, const uint32_t *query_positions,
                               const uint32_t *seq_of_row, const uint32_t *block_tables_flat,
                               const uint64_t *block_table_offsets, uint64_t num_sequences, float *out) {
  clear_error();
  ORION_TRY(check_backend(backend));
  if (num_kv_heads == 0 || num_query_heads % num_kv_heads != 0)  // attention.rs:244-248
    return set_error(ORION_ERR_INTERNAL, "%llu query heads cannot be grouped over %llu kv heads",
                     (unsigned long long)num_query_heads, (unsigned long long)num_kv_heads);
  if (block_size == 0 || head_dim == 0) return set_error(ORION_ERR_INTERNAL, "block_size and head_dim must be non-zero");
  for (uint64_t r = 0; r < rows; ++r) {
    if (seq_of_row[r] >= num_sequences) return set_error(ORION_ERR_INTERNAL, "row %llu names sequence %u of %llu",
                                                        (unsigned long long)r, seq_of_row[r], (unsigned long long)num_sequences);
    const uint64_t t0 = block_table_offsets[seq_of_row[r]], tlen = block_table_offsets[seq_of_row[r] + 1] - t0;
    const uint64_t need = (uint64_t)query_positions[r] / block_size + 1;
    if (need > tlen)  // attention.rs:263-268
      return set_error(ORION_ERR_INTERNAL, "position %u is outside the block table of %llu blocks", query_positions[r],
                       (unsigned long long)tlen);
    for (uint64_t e = 0; e < need; ++e)
      if (block_tables_flat[t0 + e] >= num_blocks)  // attention.rs:150-155
        return set_error(ORION_ERR_INTERNAL, "block %u out of range (have %llu)", block_tables_flat[t0 + e],
                         (unsigned long long)num_blocks);
  }
  if (rows == 0) return ORION_OK;
  if (dtype == ORION_DTYPE_F32)
    return op_attention<float>(kv, num_blocks, block_size, num_kv_heads, head_dim, query, rows, num_query_heads,
                               query_positions, seq_of_row, block_tables_flat, block_table_offsets, num_sequences, out);
  if (dtype == ORION_DTYPE_BF16)
    return op_attention<bf16>(kv, num_blocks, block_size, num_kv_heads, head_dim, query, rows, num_query_heads,
                              query_positions, seq_of_row, block_tables_flat, block_table_offsets, num_sequences, out);
  return bad_dtype(dtype);
}

int orion_cuda_linear_bench(OrionBackend *backend, uint64_t rows, uint64_t in_features, uint64_t out_features,
                            int warmup, int iterations, float *mean_ms, uint32_t *splits_used) {
  clear_error();
  ORION_TRY(check_backend(backend));
  Dev<bf16> x, w;
  Dev<float> part;
  ORION_TRY(x.alloc(rows * in_features));
  ORION_TRY(w.alloc(out_features * in_features));
  ORION_TRY(launch_fill_normal<bf16>(x.p, rows * in_features, 11, 0));
  ORION_TRY(launch_fill_normal<bf16>(w.p, out_features * in_features, 12, 0));
  GemmPlan p = gemm_plan(true, (uint32_t)rows, (uint32_t)out_features, (uint32_t)in_features,
                         (uint32_t)in_features, (uint32_t)in_features);
  if (!p.tensor_core) return set_error(ORION_ERR_INVALID_REQUEST, "shape is not covered by the tensor-core GEMM");
  ORION_TRY(part.alloc((size_t)p.splits * rows * out_features));
  cudaEvent_t e0, e1;
  ORION_CUDA_CHECK("create event", cudaEventCreate(&e0));
  ORION_CUDA_CHECK("create event", cudaEventCreate(&e1));
  int rc = ORION_OK;
  for (int i = 0; i < warmup + iterations && rc == ORION_OK; ++i) {
    if (i == warmup) cudaEventRecord(e0, 0);
    rc = launch_gemm<bf16>(x.p, (uint32_t)in_features, w.p, (uint32_t)in_features, part.p, (uint32_t)rows,
                           (uint32_t)out_features, (uint32_t)in_features, p, 0);
  }
  cudaEventRecord(e1, 0);
  cudaError_t e = cudaEventSynchronize(e1);
  float ms = 0.f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  ORION_TRY(rc);
  ORION_CUDA_CHECK("linear bench", e);
  uint32_t code = 0;
  ORION_TRY(gemm_tc_poll_error(&code));
  if (code) return set_error(ORION_ERR_BACKEND, "backend cuda failed at gemm: a bounded pipeline wait ran out (code %u)", code);
  if (mean_ms) *mean_ms = iterations > 0 ? ms / iterations : 0.f;
  if (splits_used) *splits_used = p.splits;
  return ORION_OK;
}

int orion_cuda_argmax(OrionBackend *backend, const float *logits, uint64_t rows, uint64_t cols, uint32_t *out) {
  clear_error();
  ORION_TRY(check_backend(backend));
  if (rows == 0) return ORION_OK;
  Dev<float> l;
  Dev<uint32_t> o;
  ORION_TRY(l.upload(logits, rows * cols));
  ORION_TRY(o.alloc(rows));
  ORION_TRY(launch_argmax(l.p, (uint32_t)rows, (uint32_t)cols, o.p, 0));
  ORION_CUDA_CHECK("argmax", cudaMemcpy(out, o.p, rows * sizeof(uint32_t), cudaMemcpyDeviceToHost));
  return ORION_OK;
}

// ---- paged decode attention microbenchmark -----------------------------------------

int orion_cuda_attn_bench_create(OrionBackend *backend, uint32_t num_query_heads, uint32_t num_kv_heads,
                                 uint32_t head_dim, uint32_t block_size, uint64_t num_blocks,
                                 const uint32_t *block_ids, const uint64_t *context_lens, uint32_t batch,
                                 uint64_t seed, OrionAttnBench **out) {
  clear_error();
  if (!out) return set_error(ORION_ERR_INVALID_REQUEST, "null output pointer");
  *out = nullptr;
  ORION_TRY(check_backend(backend));
  std::unique_ptr<OrionAttnBench> b(new OrionAttnBench());
  b->backend = backend;
  b->lay = KvLayout{1, (uint32_t)num_blocks, num_kv_heads, block_size, head_dim, head_dim % 64 == 0 ? 1u : 0u};
  b->q_heads = num_query_heads;
  b->batch = batch;
  if (!decode_attention_supported(b->lay, num_query_heads))
    return set_error(ORION_ERR_INVALID_REQUEST, "the decode attention kernel covers head_dim 128, block 16, group <= 8");
  b->offsets.assign(batch + 1, 0);
  std::vector<uint32_t> pos(batch), seq(batch);
  uint64_t total_tokens = 0, total_entries = 0;
  for (uint32_t s = 0; s < batch; ++s) {
    if (context_lens[s] == 0) return set_error(ORION_ERR_INVALID_REQUEST, "context length 0 for sequence %u", s);
    const uint64_t nb = (context_lens[s] + block_size - 1) / block_size;
    b->offsets[s + 1] = b->offsets[s] + (uint32_t)nb;
    pos[s] = (uint32_t)(context_lens[s] - 1);
    seq[s] = s;
    b->max_position = std::max(b->max_position, pos[s]);
    total_tokens += context_lens[s];
    total_entries += nb;
    b->ctx.push_back((uint32_t)context_lens[s]);
  }
  b->tables.assign(block_ids, block_ids + total_entries);
  for (uint32_t id : b->tables)
    if (id >= num_blocks) return set_error(ORION_ERR_INTERNAL, "block %u out of range (have %llu)", id, (unsigned long long)num_blocks);
  const size_t arena_n = b->lay.layer_elems(), qn = (size_t)batch * num_query_heads * head_dim;
  ORION_CUDA_CHECK("allocate arena", cudaMalloc(reinterpret_cast<void **>(&b->arena), arena_n * sizeof(bf16)));
  ORION_CUDA_CHECK("allocate", cudaMalloc(reinterpret_cast<void **>(&b->q), qn * sizeof(bf16)));
  ORION_CUDA_CHECK("allocate", cudaMalloc(reinterpret_cast<void **>(&b->out), qn * sizeof(bf16)));
  ORION_TRY(launch_fill_normal<bf16>(b->arena, arena_n, seed, 0));
  ORION_TRY(launch_fill_normal<bf16>(b->q, qn, seed ^ 0xabcdef12345ull, 0));
  std::vector<uint32_t> meta;
  meta.insert(meta.end(), pos.begin(), pos.end());
  meta.insert(meta.end(), seq.begin(), seq.end());
  meta.insert(meta.end(), b->offsets.begin(), b->offsets.end());
  meta.insert(meta.end(), b->tables.begin(), b->tables.end());
  ORION_CUDA_CHECK("allocate", cudaMalloc(reinterpret_cast<void **>(&b->meta), meta.size() * sizeof(uint32_t)));
  ORION_CUDA_CHECK("upload", cudaMemcpy(b->meta, meta.data(), meta.size() * sizeof(uint32_t), cudaMemcpyHostToDevice));
  {
    const DecodePlan plan = decode_plan(batch, num_kv_heads, total_entries, b->max_position, block_size, 32);
    b->splits = plan.splits;
    b->blocks_per_split = plan.blocks_per_split;
  }
  const size_t scratch_bytes = decode_scratch_floats(batch, num_query_heads, head_dim, b->splits) * sizeof(float);
  ORION_CUDA_CHECK("allocate", cudaMalloc(reinterpret_cast<void **>(&b->scratch), scratch_bytes));
  ORION_CUDA_CHECK("clear attention scratch", cudaMemset(b->scratch, 0, scratch_bytes));
  // K and V once per kv head and context token, q in and out once, one table entry per block.
  b->algorithmic_bytes = total_tokens * num_kv_heads * head_dim * 2 * 2 + (uint64_t)qn * 2 * 2 + total_entries * 4;
  ORION_CUDA_CHECK("create event", cudaEventCreate(&b->ev0));
  ORION_CUDA_CHECK("create event", cudaEventCreate(&b->ev1));
  ORION_CUDA_CHECK("attn bench", cudaDeviceSynchronize());
  *out = b.release();
  return ORION_OK;
}

static int attn_bench_launch(OrionAttnBench *b) {
  const uint32_t n = b->batch;
  AttnBatch ab{b->meta, b->meta + n, b->meta + 2 * n + (n + 1), b->meta + 2 * n, n, b->max_position};
  DecodeScratch sc = decode_scratch_at(b->scratch, n, b->q_heads, b->lay.num_kv_heads, b->lay.head_dim, b->splits,
                                       b->blocks_per_split);
  return launch_paged_attention_decode(b->q, b->arena, b->lay, 0, ab, b->q_heads, b->splits, sc, b->out, 0);
}

int orion_cuda_attn_bench_run(OrionAttnBench *bench, int warmup, int iterations, float *mean_ms,
                              uint64_t *algorithmic_bytes) {
  clear_error();
  if (!bench) return set_error(ORION_ERR_INVALID_REQUEST, "null bench handle");
  ORION_TRY(check_backend(bench->backend));
  for (int i = 0; i < warmup; ++i) ORION_TRY(attn_bench_launch(bench));
  ORION_CUDA_CHECK("attn bench", cudaDeviceSynchronize());
  ORION_CUDA_CHECK("attn bench", cudaEventRecord(bench->ev0, 0));
  for (int i = 0; i < iterations; ++i) ORION_TRY(attn_bench_launch(bench));
  ORION_CUDA_CHECK("attn bench", cudaEventRecord(bench->ev1, 0));
  ORION_CUDA_CHECK("attn bench", cudaEventSynchronize(bench->ev1));
  float ms = 0.f;
  ORION_CUDA_CHECK("attn bench", cudaEventElapsedTime(&ms, bench->ev0, bench->ev1));
  if (mean_ms) *mean_ms = iterations > 0 ? ms / iterations : 0.f;
  if (algorithmic_bytes) *algorithmic_bytes = bench->algorithmic_bytes;
  uint32_t code = 0;
  ORION_TRY(decode_poll_error(&code));
  if (code) return set_error(ORION_ERR_BACKEND, "backend cuda failed at attention: a bounded pipeline wait ran out (code %u)", code);
  return ORION_OK;
}

int orion_cuda_attn_bench_output(OrionAttnBench *bench, float *out) {
  clear_error();
  if (!bench || !out) return set_error(ORION_ERR_INVALID_REQUEST, "null pointer argument");
  ORION_TRY(check_backend(bench->backend));
  const size_t qn = (size_t)bench->batch * bench->q_heads * bench->lay.head_dim;
  Dev<float> f;
  ORION_TRY(f.alloc(qn));
  ORION_TRY(launch_convert_to_f32<bf16>(bench->out, f.p, qn, 0));
  ORION_CUDA_CHECK("attn bench", cudaMemcpy(out, f.p, qn * sizeof(float), cudaMemcpyDeviceToHost));
  return ORION_OK;
}

int orion_cuda_attn_bench_sequence(OrionAttnBench *bench, uint32_t seq, float *q, float *k, float *v) {
  clear_error();
  if (!bench || !q || !k || !v) return set_error(ORION_ERR_INVALID_REQUEST, "null pointer argument");
  if (seq >= bench->batch) return set_error(ORION_ERR_INVALID_REQUEST, "sequence %u of %u", seq, bench->batch);
  ORION_TRY(check_backend(bench->backend));
  const KvLayout &lay = bench->lay;
  const uint32_t hd = lay.head_dim, B = lay.block_size, H = lay.num_kv_heads;
  const size_t qn = (size_t)bench->q_heads * hd;
  std::vector<uint16_t> hq(qn);
  ORION_CUDA_CHECK("attn bench", cudaMemcpy(hq.data(), bench->q + (size_t)seq * qn, qn * 2, cudaMemcpyDeviceToHost));
  auto widen = [](uint16_t bits) { uint32_t w = (uint32_t)bits << 16; float f; std::memcpy(&f, &w, 4); return f; };
  for (size_t i = 0; i < qn; ++i) q[i] = widen(hq[i]);
  const uint32_t ctx = bench->ctx[seq];
  std::vector<uint16_t> chunk(lay.chunk_elems());
  for (uint32_t lb = 0; lb * B < ctx; ++lb) {
    const uint32_t pb = bench->tables[bench->offsets[seq] + lb];
    for (uint32_t h = 0; h < H; ++h) {
      ORION_CUDA_CHECK("attn bench", cudaMemcpy(chunk.data(), bench->arena + ((size_t)pb * H + h) * lay.chunk_elems(),
                                                chunk.size() * 2, cudaMemcpyDeviceToHost));
      for (uint32_t slot = 0; slot < B && lb * B + slot < ctx; ++slot) {
        const size_t t = (size_t)lb * B + slot;
        for (uint32_t d = 0; d < hd; ++d) {
          k[(t * H + h) * hd + d] = widen(chunk[(size_t)slot * hd + lay.col(slot, d)]);
          v[(t * H + h) * hd + d] = widen(chunk[((size_t)B + slot) * hd + lay.col(slot, d)]);
        }
      }
    }
  }
  return ORION_OK;
}

int orion_cuda_attn_bench_device_views(OrionAttnBench *bench, const void **q, const void **kv_arena,
                                       const uint32_t **query_positions, const uint32_t **seq_of_row,
                                       const uint32_t **block_tables_flat, const uint32_t **block_table_offsets,
                                       uint32_t *max_position) {
  clear_error();
  if (!bench) return set_error(ORION_ERR_INVALID_REQUEST, "null bench handle");
  const uint32_t n = bench->batch;
  if (q) *q = bench->q;
  if (kv_arena) *kv_arena = bench->arena;
  if (query_positions) *query_positions = bench->meta;
  if (seq_of_row) *seq_of_row = bench->meta + n;
  if (block_table_offsets) *block_table_offsets = bench->meta + 2 * n;
  if (block_tables_flat) *block_tables_flat = bench->meta + 2 * n + (n + 1);
  if (max_position) *max_position = bench->max_position;
  return ORION_OK;
}

void orion_cuda_attn_bench_destroy(OrionAttnBench *bench) { delete bench; }

}  // extern "C"
