// The tail of a greedy generation step in one launch: arg-max over the logits of every sequence,
// the new token written to its column of the output ids, the embedding of that token for the
// NEXT step (word + position), and the step's position scalars advanced.
//
// Replaces, per step, the reference's `torch.argmax` / `torch.cat` / `self.embed(...)` sequence
// (energonai/model/model_factory.py:124-131, energonai/model/embedding.py:44-57), which as separate
// framework kernels is nine launches of a few microseconds each on the critical path of a step
// that is itself a chain of short launches.
//
// One CTA per sequence.  The position scalars are read by every CTA before it reports in; the
// last CTA to report in advances them (so the launches of the next step find them advanced) and
// rearms the counter.
#include <cfloat>

#include "common.cuh"

namespace eb {
namespace {

constexpr int kStepThreads = 256;

struct StepParams {
  const void *logits;          // [batch][ld_logits], T
  long long ld_logits;
  int batch, vocab;
  long long *out_ids;          // [batch][ld_out]
  long long ld_out;
  int out_cols;                // columns of out_ids that may be written
  long long *tok;              // [batch] or null
  int *kv_state;               // [0] position of the token just processed, [1] column of the new token
  const void *word_emb;        // [vocab_rows][hidden] T or null (then no embedding is produced)
  long long vocab_start;       // first token id held in word_emb (vocabulary split over ranks)
  int vocab_rows;
  const void *pos_emb;         // [pos_rows][hidden] T
  int pos_rows, add_pos;       // add_pos: this rank contributes the position embedding
  int hidden;
  void *hidden_out;            // [batch][ld_hidden] T
  long long ld_hidden;
  int *counter;                // zero between launches
};

// L: type of the logits, T: type of the embedding tables and of the output row
template <typename L, typename T>
__global__ void __launch_bounds__(kStepThreads) greedy_step_kernel(const StepParams p) {
  __shared__ float s_val[kStepThreads / 32];
  __shared__ int s_idx[kStepThreads / 32];
  __shared__ int s_token;
  griddep_wait();
  griddep_launch();
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pos = p.kv_state[0], col = p.kv_state[1];
  const L *row = reinterpret_cast<const L *>(p.logits) + (long long)b * p.ld_logits;

  // arg-max, the lowest index among equal maxima
  float best = -FLT_MAX;
  int best_i = 0x7fffffff;
  auto take = [&](float v, int i) {
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  };
  constexpr int VEC = 16 / sizeof(L);
  if ( p.ld_logits % VEC == 0 && (reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
    const int packs = p.vocab / VEC;
    for (int v = tid; v < packs; v += kStepThreads) {
      Vec16<L> pk;
      pk.load(row + (long long)v * VEC);
      float f[VEC];
      pk.unpack(f);
#pragma unroll
      for (int e = 0; e < VEC; ++e) take(f[e], v * VEC + e);
    }
    for (int i = packs * VEC + tid; i < p.vocab; i += kStepThreads) take(to_f32<L>(row[i]), i);
  } else {
    for (int i = tid; i < p.vocab; i += kStepThreads) take(to_f32<L>(row[i]), i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    take(ov, oi);
  }
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = lane < kStepThreads / 32 ? s_val[lane] : -FLT_MAX;
    best_i = lane < kStepThreads / 32 ? s_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      take(ov, oi);
    }
    if (lane == 0) {
      const int token = best_i == 0x7fffffff ? 0 : best_i;      // a row of NaNs: token 0
      s_token = token;
      if (p.tok) p.tok[b] = token;
      if (col >= 0 && col < p.out_cols) p.out_ids[(long long)b * p.ld_out + col] = token;
    }
  }
  __syncthreads();
  const int token = s_token;

  // embedding of the new token at the next position
  if (p.word_emb) {
    const long long local = (long long)token - p.vocab_start;
    const bool mine = local >= 0 && local < p.vocab_rows;
    const int next = pos + 1 < p.pos_rows ? pos + 1 : p.pos_rows - 1;
    const T *w = reinterpret_cast<const T *>(p.word_emb) + (mine ? local : 0) * p.hidden;
    const T *q = reinterpret_cast<const T *>(p.pos_emb) + (long long)next * p.hidden;
    T *o = reinterpret_cast<T *>(p.hidden_out) + (long long)b * p.ld_hidden;
    for (int d = tid; d < p.hidden; d += kStepThreads) {
      const float wv = mine ? to_f32<T>(w[d]) : 0.f, pv = p.add_pos ? to_f32<T>(q[d]) : 0.f;
      o[d] = from_f32<T>(wv + pv);
    }
  }

  // every CTA has read the position scalars: the last one advances them
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(p.counter, 1) == (int)gridDim.x - 1) {
      p.kv_state[0] = pos + 1;
      p.kv_state[1] = col + 1;
      *p.counter = 0;
      __threadfence();
    }
  }
}

}  // namespace
}  // namespace eb

using namespace eb;

namespace {
template <typename L>
void launch_step(int emb_dtype, int batch, cudaStream_t st, const StepParams &p) {
  if (emb_dtype == EB_F32) launch_pdl(greedy_step_kernel<L, float>, dim3(batch), dim3(kStepThreads), 0, st, p);
  else if (emb_dtype == EB_F16) launch_pdl(greedy_step_kernel<L, __half>, dim3(batch), dim3(kStepThreads), 0, st, p);
  else launch_pdl(greedy_step_kernel<L, __nv_bfloat16>, dim3(batch), dim3(kStepThreads), 0, st, p);
}
}  // namespace

extern "C" int eb_greedy_step(const void *logits, long long ld_logits, int batch, int vocab, int dtype, int64_t *out_ids,
                              long long ld_out, int out_cols, int64_t *tok, int32_t *kv_state, const void *word_emb,
                              long long vocab_start, int vocab_rows, const void *pos_emb, int pos_rows, int add_pos, int hidden,
                              int emb_dtype, void *hidden_out, long long ld_hidden, int32_t *counter, void *stream) {
  if (batch == 0) return EB_OK;
  EB_REQUIRE(dtype_ok(dtype) && (!word_emb || dtype_ok(emb_dtype)), "greedy_step: bad dtype %d / %d", dtype, emb_dtype);
  EB_REQUIRE(batch > 0 && batch <= 65535 && vocab > 0, "greedy_step: bad batch %d or vocabulary %d", batch, vocab);
  EB_REQUIRE(logits && out_ids && kv_state && counter, "greedy_step: null pointer");
  EB_REQUIRE(ld_logits >= vocab && ld_out >= out_cols && out_cols >= 0, "greedy_step: leading dimensions smaller than the rows they hold");
  if (word_emb) {
    EB_REQUIRE(pos_emb && hidden_out && hidden > 0 && vocab_rows > 0 && pos_rows > 0 && ld_hidden >= hidden,
               "greedy_step: the embedding needs word and position tables, an output and their sizes");
  }
  StepParams p{};
  p.logits = logits; p.ld_logits = ld_logits; p.batch = batch; p.vocab = vocab;
  p.out_ids = reinterpret_cast<long long *>(out_ids); p.ld_out = ld_out; p.out_cols = out_cols;
  p.tok = reinterpret_cast<long long *>(tok); p.kv_state = kv_state;
  p.word_emb = word_emb; p.vocab_start = vocab_start; p.vocab_rows = vocab_rows;
  p.pos_emb = pos_emb; p.pos_rows = pos_rows; p.add_pos = add_pos; p.hidden = hidden;
  p.hidden_out = hidden_out; p.ld_hidden = ld_hidden; p.counter = counter;
  cudaStream_t st = as_stream(stream);
  if (!word_emb) emb_dtype = EB_F16;
  if (dtype == EB_F32) launch_step<float>(emb_dtype, batch, st, p);
  else if (dtype == EB_F16) launch_step<__half>(emb_dtype, batch, st, p);
  else launch_step<__nv_bfloat16>(emb_dtype, batch, st, p);
  return check_launch("greedy_step");
}
