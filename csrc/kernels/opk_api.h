// C ABI of libopake_kernels.so. Every entry point takes raw device pointers and a CUDA stream, allocates
// nothing unless stated, and returns a cudaError_t-compatible int (0 = success; negative = argument error).
// The Python side (opake_b200/ops/_lib.py) binds these with ctypes.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct OpkGemmArgs {
  const void* A;       // bf16
  const void* B;       // bf16
  void* C;             // bf16 output (unused for epilogue 3)
  const void* R;       // optional residual (same layout as C)
  const void* bias;    // optional bf16 [N]
  int32_t M, N, K, batch;
  int32_t a_mn;        // 0: A is [M][K] (lda = row pitch); 1: A is [K][M]
  int32_t b_mn;        // 0: B is [N][K];                   1: B is [K][N]
  int32_t epilogue;    // GemmEpilogue
  int32_t b_batch_div; // B batch index = b / b_batch_div
  int64_t lda, ldb, ldc;                 // row pitches in elements
  int64_t strideA, strideB, strideC;     // batch strides in elements
  float alpha;
  float softcap;
  double* sumsq;       // epilogue 1
  void* act;           // epilogue 2
  int64_t ld_act;
  const int32_t* labels;  // epilogue 3/4
  float* pmax;
  float* psum;
  float* tgt;
  const float* lse;
  const float* coef;
  int32_t* err;        // device int, set to 1 if a bounded wait expired
  int32_t max_ctas;    // 0 = one per SM
  // grouped modes (see GemmParams in gemm_sm100.cuh); all optional
  const int32_t* tile_group;  // device [ceil(M/128)]: group of every 128-row tile of A / C, -1 = skip; B has n_groups batches
  int32_t n_groups;
  const int32_t* group_k;     // device [batch][2]: {first reduction element, number of 64-element blocks} per batch entry
  int32_t sumsq_shared;       // epilogue 1: every batch entry adds into sumsq[0]
  // Staged B (see opk_gemm): B is another GPU's memory; stage_dst = local scratch [N][K] bf16, stage_ready = int32
  // counters, one per band of 2048 rows of B (zeroed by opk_gemm on the stream before the launch).
  void* stage_dst;
  int32_t* stage_ready;
} OpkGemmArgs;

int opk_gemm(const OpkGemmArgs* args, void* stream);
int opk_gemm_tiles_n(int N, int epilogue);  // number of column tiles the kernel uses (LCE partial buffers)
int opk_num_sms(void);
// Two-CTA (cta_group::2) kernel for eligible products: on by default, OPK_GEMM_PAIR=0 or set_pair_mode(0) turns it off.
void opk_gemm_set_pair_mode(int on);
int opk_gemm_get_pair_mode(void);
// Debug-build index checks (library variant built with OPK_DEBUG_BOUNDS): out4 = {failing accesses since the last reset,
// source line of the first, its index, its bound}; file_out receives the first record's source file. Synchronises the
// device. Returns -3 from a release build. A failing access is skipped by the kernel, never performed.
int opk_debug_bounds_read(int64_t* out4, char* file_out, int file_cap, int reset);
// Bounded-wait self-test: one CTA waits `budget_cycles` on a barrier nobody completes, then sets *err = 3 and returns.
int opk_wait_selftest(int32_t* err, int64_t budget_cycles, int64_t* waited_cycles, void* stream);
const char* opk_last_error(void);

// ---- normalisation / rotary / activation / embedding (csrc/kernels/elementwise.cu) -------------------------
// y = x * rsqrt(mean(x^2) + eps) * (w + offset); rstd[T] saved for backward. x, y, w bf16.
int opk_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int T, int D, float eps, float w_offset,
                    void* stream);
// The same with row pitches (elements): normalises a column slice of a wider matrix, e.g. the query part of a fused
// QKV activation. x and y may alias.
int opk_rmsnorm_fwd_ld(const void* x, int64_t ldx, const void* w, void* y, int64_t ldy, float* rstd, int T, int D, float eps,
                       float w_offset, void* stream);
int opk_rmsnorm_bwd_ld(const void* dy, int64_t ld_dy, const void* x, int64_t ldx, const void* w, const float* rstd,
                       const void* dres, void* dx_out, int64_t ld_dx, float* dw, float* workspace, int ws_rows, int T, int D,
                       float w_offset, void* stream);
// s = x + r (stored to sum_out), then RMSNorm of s.
int opk_add_rmsnorm_fwd(const void* x, const void* r, const void* w, void* sum_out, void* y, float* rstd, int T, int D,
                        float eps, float w_offset, void* stream);
// dx_out = dres (optional) + d(rmsnorm)/dx ; dw[D] (fp32) += sum_t dy * xhat.  dw must be zeroed by the caller.
// workspace: fp32 [ws_rows][D] scratch for per-CTA partial weight gradients (needed when dw is given; 296 rows
// let the kernel use its full grid). Calls that share a workspace must be ordered on one stream.
int opk_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx_out,
                    float* dw, float* workspace, int ws_rows, int T, int D, float w_offset, void* stream);
// LayerNorm (GPT-2): y = (x - mean) * rstd * w + b
int opk_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int T, int D,
                      float eps, void* stream);
int opk_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                      const void* dres, void* dx_out, float* dw, float* db, int T, int D, void* stream);
// In-place rotary embedding on the first n_rot_heads heads of each row (heads are head_dim wide, row pitch ld).
// cs = [T][head_dim/2][2] fp32 (cos, sin); pos = optional int32 [T] row -> table row. sign = +1 forward, -1 backward.
int opk_rope(void* qk, const float* cs, const int32_t* pos, int T, int n_rot_heads, int head_dim, int64_t ld,
             float sign, void* stream);
// SwiGLU on interleaved (gate, up) columns. fwd: act[T][F]; bwd: dgu[T][2F] from dact[T][F] and gu[T][2F].
int opk_swiglu_fwd(const void* gu, void* act, int T, int F, void* stream);
int opk_swiglu_bwd(const void* dact, const void* gu, void* dgu, int T, int F, void* stream);
// GEGLU (tanh approximation when approx != 0), same interleaved layout.
int opk_geglu_fwd(const void* gu, void* act, int T, int F, int approx, void* stream);
int opk_geglu_bwd(const void* dact, const void* gu, void* dgu, int T, int F, int approx, void* stream);
// GELU (GPT-2 "gelu_new" tanh form): y = gelu(x); backward dx = dy * gelu'(x).
int opk_gelu_fwd(const void* x, void* y, int64_t n, void* stream);
int opk_gelu_bwd(const void* dy, const void* x, void* dx, int64_t n, void* stream);
// out[t] = table[tok[t]] (+ pos_table[t] when given)
int opk_embedding_fwd(const int32_t* tok, const void* table, const void* pos_table, void* out, int T, int D, int vocab,
                      void* stream);
// Per-example embedding gradient without a dense [V][D] buffer: rows with equal tokens are summed into the row of
// their first occurrence. first_pos is an int32 [V] scratch that must hold INT32_MAX on entry and is restored.
// Outputs: rep[T] (first position of the same token), gc[T][D] fp32 (zeroed here), sumsq += sum(bf16(gc)^2).
// vocab is the length of first_pos; a token id outside [0, vocab) is skipped (rep[t] = -1, no row written).
int opk_embedding_bwd_compact(const int32_t* tok, const void* dx, int32_t* first_pos, int32_t* rep, float* gc,
                              double* sumsq, int T, int D, int vocab, void* stream);
// acc[tok[t]] += bf16(gc[t] * scale) for the representative rows (rep[t] == t).
int opk_embedding_accumulate(const int32_t* tok, const int32_t* rep, const float* gc, const float* scale, float* acc,
                             int T, int D, void* stream);
// Same, with reductions (red.add) instead of read-modify-write: for an acc whose rows other GPUs add to at the same time
// (sharded sums; acc may be the peer-mapped shard of the rank that owns the embedding table).
int opk_embedding_accumulate_shared(const int32_t* tok, const int32_t* rep, const float* gc, const float* scale, float* acc,
                                    int T, int D, void* stream);
// Fused linear-cross-entropy finalisation: lse[t] from the per-tile partials, nll[t] = lse - tgt (0 if ignored).
int opk_lce_finalize(const float* pmax, const float* psum, const float* tgt, const int32_t* labels, float* lse,
                     float* nll, int T, int tiles, void* stream);
// Per-example RMSNorm weight gradients under a batched (vmapped) backward: dy, x are [B * rows][D] bf16 (example b owns
// rows b*rows .. (b+1)*rows - 1), rstd [B * rows]; dw [B][D] fp32 is ACCUMULATED into (zero it first).
int opk_rmsnorm_dw_per_example(const void* dy, const void* x, const float* rstd, float* dw, int B, int rows, int D, void* stream);
// Per-example loss bookkeeping: ntok = max(1, number of labels >= 0); coef[t] = (label >= 0) / ntok, times *weight when
// weight != NULL; *loss = sum_t nll[t] * coef[t]; *ntok (may be NULL) = ntok. One CTA.
int opk_loss_coef(const int32_t* labels, const float* nll, const float* weight, float* coef, float* loss, float* ntok, int T,
                  void* stream);
// Row-wise cross entropy over materialised logits (bf16 or fp32): nll[t], optional lse[t]; softcap / scale as LCE.
int opk_cross_entropy_fwd(const void* logits, int is_fp32, const int32_t* labels, float* nll, float* lse, int T, int V,
                          int64_t ld, float scale, float softcap, void* stream);
int opk_cross_entropy_bwd(const void* logits, int is_fp32, const int32_t* labels, const float* lse, const float* coef,
                          void* dlogits, int T, int V, int64_t ld, float scale, float softcap, void* stream);
// sum(x^2) of a bf16/fp32 vector (x rounded to bf16 first when round_bf16) added to *sumsq (double).
int opk_sumsq(const void* x, int is_fp32, int round_bf16, int64_t n, double* sumsq, void* stream);
// fp32 rows -> bf16 at dst_base + offsets[r] (device int64 array), with sum of squares of the stored values.
int opk_scatter_rows_cast_sumsq(const float* src, void* dst_base, const int64_t* offsets, int R, int D, double* sumsq,
                                void* stream);
// out[n] += sum_t dy[t][n] (out fp32, zeroed by the caller)
int opk_colsum(const void* dy, float* out, int T, int N, int64_t ld, void* stream);
// Tied embeddings: dense[tok[t]] += gc[t] for first-occurrence rows (bf16 read-modify-write).
int opk_embedding_add_rows(const int32_t* tok, const int32_t* rep, const float* gc, void* dense, int T, int D,
                           void* stream);
// out_bf16 = bf16(in_fp32)
int opk_cast_f32_bf16(const float* in, void* out, int64_t n, void* stream);

// ---- causal GQA flash attention on the fused projection buffer (csrc/kernels/attention_sm100.cu) -------------
// qkv bf16 [T][(H+2KV)*hd] (row pitch ld), out bf16 [T][H*hd] (row pitch ldo), lse fp32 [H][T]. hd in {64, 128}.
int opk_attn_fwd(const void* qkv, void* out, float* lse, int T, int H, int KV, int hd, int64_t ld, int64_t ldo,
                 float scale, int32_t* err, void* stream);
// Backward: dqkv (same layout as qkv) receives dQ, dK, dV. dsum is a 16-byte-aligned fp32 work buffer of
// 2 * H * T64 elements, T64 = T rounded up to a multiple of 64 (rowsum(dO * O), then -lse * log2 e).
// part (optional, 16-byte aligned, 2 * (H/KV) * T * KV*hd floats): with grouped-query attention the dK / dV kernel
// then runs one CTA per query head, writes fp32 partials there and a reduce kernel sums them in a fixed order.
int opk_attn_bwd(const void* qkv, const void* out, const void* dout, const float* lse, float* dsum, void* dqkv,
                 float* part, int T, int H, int KV, int hd, int64_t ld, int64_t ldo, float scale, int32_t* err,
                 void* stream);

// ---- multi-tensor clip-and-sum of materialised per-example gradients (csrc/kernels/clip_sum.cu) -----------------
// `tiles`: device array of n_tiles descriptors {const void* base; float* out; int64 n; int64 off; int32 is_bf16; int32 pad}
// (opk_clip_sum_desc_bytes() bytes each), one per opk_clip_sum_tile() elements of one example of one leaf.
int opk_clip_sum_tile(void);
int opk_clip_sum_desc_bytes(void);
// partial[b][tile] = sum of squares (fp32 squares, fp64 sum) of that tile of example b.
int opk_clip_sumsq_partial(const void* tiles, int n_tiles, int B, double* partial, void* stream);
// out[i] = sum_b stored(g_b[i] * f[b]) per leaf; post_partial (optional) [b][tile] = squared norm after clipping.
int opk_clip_apply_sum(const void* tiles, int n_tiles, int B, const float* f_bf16, const float* f_fp32,
                       double* post_partial, void* stream);

// ---- expert-parallel dispatch / combine over peer memory (csrc/kernels/ep.cu) ------------------------------------
#define OPK_EP_MAX_RANKS 8
#define OPK_EP_PHASES 7
#define OPK_EP_PHASE_COUNTS 0   // routing histograms have been stored into the peers' control blocks
#define OPK_EP_PHASE_ROWS 1     // forward rows have been stored into the owners' receive buffers
#define OPK_EP_PHASE_OUT 2      // expert outputs are complete in the owner's buffer
#define OPK_EP_PHASE_DROWS 3    // backward: upstream-gradient rows have been stored
#define OPK_EP_PHASE_DOUT 4     // backward: input-gradient rows are complete in the owner's buffer
#define OPK_EP_PHASE_BARRIER 5  // plain group barrier (buffer reuse)
#define OPK_EP_PHASE_SUMS 6     // small all-reduce: every rank's vector has been stored into the peers' slots
typedef struct {
  int32_t world, rank, n_experts;
  int32_t r_cap;                      // rows of every rank's row buffers (multiple of 128)
  void* ctrl[OPK_EP_MAX_RANKS];       // device address of every rank's control block (opk_ep_ctrl_ints int32, zeroed once)
  // Optional device int32[2]: {base of the exchange epochs, base of the barrier epochs}. Every `epoch` argument below is
  // then RELATIVE to the base read on the device, so a captured launch sequence (frozen arguments) can be replayed:
  // opk_ep_advance moves the bases forward at the end of the sequence. Null: epochs are absolute.
  const int32_t* epoch_base;
} OpkEpGroup;
typedef struct { void* p[OPK_EP_MAX_RANKS]; } OpkEpPeers;   // the same row buffer on every rank
int opk_ep_ctrl_ints(int world, int n_experts);
int opk_ep_rows_capacity(int world, int n_entries, int n_experts);
// entry_rank[n] = stable rank of entry n among this rank's entries of the same expert; histogram pushed to all peers.
int opk_ep_count(const OpkEpGroup* g, const int32_t* idx, int n_entries, int32_t* entry_rank, int epoch, void* stream);
// Stores row (n / k) of x (times entry_scale[n]) into its slot on the owner. replay = 0: slots derived from the
// histograms (entry_pos written: owner << 26 | row); replay = 1: slots read from entry_pos (backward pass).
int opk_ep_dispatch(const OpkEpGroup* g, const OpkEpPeers* rows, const void* x, int64_t ldx, int k, const float* entry_scale,
                    const int32_t* idx, const int32_t* entry_rank, int32_t* entry_pos, int replay, int n_entries, int D,
                    int wait_phase, int signal_phase, int epoch, int32_t* err, void* stream);
// Owner side: tile -> local expert table [r_cap / 128], reduction ranges per local expert [E_local][2] and per
// (local expert, source) [E_local * world][2], row -> source table [r_cap] (-1 = padding), number of rows in use.
int opk_ep_prepare(const OpkEpGroup* g, int wait_phase, int epoch, int32_t* tile_group, int32_t* group_k_expert,
                   int32_t* group_k_src, int32_t* row_src, int32_t* rows_total, int32_t* err, void* stream);
int opk_ep_zero_pad(void* rows, const int32_t* row_src, const int32_t* rows_total, int r_cap, int D, void* stream);
int opk_ep_scale_rows(const void* rows, const int32_t* row_src, const float* scale, int r_cap, int D, void* out, void* stream);
int opk_ep_signal(const OpkEpGroup* g, int phase, int epoch, void* stream);
// epoch_base[0] += d_epoch, epoch_base[1] += d_barrier (one thread; stream-ordered after the sequence that used them).
int opk_ep_advance(int32_t* epoch_base, int d_epoch, int d_barrier, void* stream);
// out[i] = sum over ranks of that rank's local[i], i < n <= 64 (fp64). `slots` is an [world][64] double buffer on
// every rank: each rank stores its vector into slot [its rank] of every peer, raises OPK_EP_PHASE_SUMS, waits (bounded)
// for all peers and adds the slots in rank order, so every rank gets the same bits.
int opk_ep_allreduce_f64(const OpkEpGroup* g, const OpkEpPeers* slots, const double* local, int n, int epoch, double* out,
                         int32_t* err, void* stream);
int opk_ep_wait(const OpkEpGroup* g, int phase, int epoch, int32_t* err, void* stream);
int opk_ep_combine(const OpkEpGroup* g, const OpkEpPeers* y, const int32_t* entry_pos, const float* wts, int k,
                   const void* residual, int T, int D, void* out, int wait_phase, int epoch, int32_t* err, void* stream);
int opk_ep_combine_bwd(const OpkEpPeers* y, const void* dy, const int32_t* entry_pos, int n_entries, int k, int D, float* dwts,
                       void* stream);

// ---- mixture-of-experts routing / permutation (csrc/kernels/moe.cu) -------------------------------------------
// probs = softmax(logits[T][E] bf16); idx / wts [T][k]: the k largest (ties: lowest expert), renormalised if norm_topk.
int opk_moe_route(const void* logits, int64_t ld, int T, int E, int k, int norm_topk, int32_t* idx, float* wts, float* probs,
                  void* stream);
int opk_moe_route_bwd(const float* probs, const int32_t* idx, const float* dwts, int T, int E, int k, int norm_topk,
                      void* dlogits, int64_t ld, void* stream);
// Worst-case number of rows of the expert-sorted buffers for n_entries = T*k routed entries.
int opk_moe_rows_capacity(int n_entries, int E);
// Stable sort of the entries by expert into 128-row aligned segments. dest[n] = row of entry n; src_entry[row] = entry
// or -1 (padding); tile_group[r_cap/128] and group_k[E][2] are the tables of the grouped GEMM modes; counts[E] optional.
int opk_moe_plan(const int32_t* idx, int n_entries, int E, int r_cap, int32_t* dest, int32_t* src_entry, int32_t* tile_group,
                 int32_t* group_k, int32_t* counts, void* stream);
// out[row] = entry_scale[n] * x[n / k] for n = src_entry[row] (zeros when n < 0); bf16 rows of D elements.
int opk_moe_gather(const void* x, int64_t ldx, const int32_t* src_entry, int k, const float* entry_scale, int R, int D, void* out,
                   void* stream);
// out[t] = residual[t] + sum_s wts[t][s] * y[dest[t][s]] (wts == NULL: plain sum).
int opk_moe_combine(const void* y, const int32_t* dest, const float* wts, int k, const void* residual, int T, int D, void* out,
                    void* stream);
// dwts[n] = <dy[n / k], y[dest[n]]>.
int opk_moe_combine_bwd(const void* dy, const void* y, const int32_t* dest, int n_entries, int k, int D, float* dwts, void* stream);

// ---- DP clipping / noise / optimizer (csrc/kernels/dp_step.cu) ---------------------------------------------
// scale = guarded min(1, C / sqrt(sumsq)) (fixed) or R / (sqrt(sumsq) + gamma) (auto); see dp_step.cu.
// Also: norm_out[0] = sqrt(sumsq), counters[0] += (norm > C), and *sumsq is reset to 0 when reset != 0.
int opk_clip_scale(double* sumsq, float clip, int mode_auto, float gamma, int n_leaves, int64_t widest_leaf,
                   float* scale_out, float* norm_out, int32_t* counters, int reset, void* stream);
// acc[i] += float(bf16(float(g[i]) * scale)) with bf16 subnormals that rounded up flushed to zero.
int opk_clip_accumulate(const void* g, const float* scale, float* acc, int64_t n, void* stream);
// Same with overwrite != 0 meaning acc = bf16(g * scale) (first example of a step: no separate zeroing pass).
int opk_clip_accumulate2(const void* g, const float* scale, float* acc, int64_t n, int overwrite, void* stream);
// A group of up to OPK_ACC_GROUP_MAX examples at once: acc (+)= sum_j stored(g[j] * *scale[j]) in one pass over acc.
// g and scale are HOST arrays of device pointers.
#define OPK_ACC_GROUP_MAX 8
int opk_clip_accumulate_group(const void* const* g, const float* const* scale, int n_group, float* acc, int64_t n, int overwrite,
                              void* stream);
// Gaussian noise from Philox4x32-10: out[i] (+)= sigma * N(0,1)_{key, stream, step, offset + i}.
int opk_philox_normal(float* out, int64_t n, uint64_t seed, uint32_t stream_id, uint32_t step, uint64_t offset,
                      float sigma, int accumulate, void* stream);

typedef struct OpkDpStepArgs {
  // gradient sources: n_src buffers (this rank's and its peers') of the fp32 clipped-gradient sum, all same layout
  const float* const* grad_src;  // device array of n_src pointers (element 0.. = ranks in rank order)
  int32_t n_src;
  int64_t shard_begin;   // first element of the global flat parameter vector owned by this rank
  int64_t shard_len;     // number of owned elements
  float inv_batch;       // 1 / normalize_by
  float sigma;           // noise std in the normalised units (noise_multiplier * C / B)
  uint64_t seed;         // RngKey.seed of the step key
  uint32_t stream_id;    // Philox stream (0 = gradient noise)
  uint32_t step;
  // optimizer state for the shard (length shard_len)
  float* m;
  float* v;
  float* master;         // optional fp32 master weights for the shard (may be NULL)
  // parameter outputs: n_dst full-size bf16 parameter buffers (own + peers); shard is written at shard_begin
  void* const* param_dst;
  int32_t n_dst;
  const void* param_src; // this rank's bf16 parameters (full-size), read when master == NULL
  float lr, beta1, beta2, eps, weight_decay;
  float bc1, bc2;        // 1 - beta^t
  float phi_hat;         // bias-corrected noise second moment (0 disables the correction)
  int32_t zero_grad;     // zero this rank's shard region in every grad_src after reading
  // optional correlated-noise (BLT) state for DP-FTRL: nbuf buffers of shard_len fp32
  float* blt_state;
  int32_t blt_nbuf;
  const float* blt_decay;  // device [nbuf]
  const float* blt_scale;  // device [nbuf]
  int32_t sgd_mode;      // 1: plain SGD update p -= lr * g (no moments)
  // optional banded-Toeplitz correlated noise (band-MF, banded square root): ring of the last toep_nlag outputs, each
  // shard_len fp32; toep_coef is a device array of toep_nlag + 1 coefficients (c_0 first). Lag k sits in ring slot
  // (toep_pos + k - 1) mod toep_nlag; the kernel overwrites slot (toep_pos - 1) mod toep_nlag, the caller's next toep_pos.
  // toep_coef != NULL with toep_nlag == 0 divides the draw by c_0 only. Exclusive with the BLT buffers.
  float* toep_state;
  int32_t toep_nlag;
  const float* toep_coef;
  int32_t toep_pos;
} OpkDpStepArgs;
int opk_dp_step(const OpkDpStepArgs* args, void* stream);

// Sharded fp32 sums ("push" reduce-scatter of one accumulation group): owner o keeps elements [bounds[o], bounds[o+1])
// of the flat vector at acc_shards[o] (peer-mapped for remote owners); the group's clipped sum is sent there with
// vector reductions. bounds: host array of n_shards + 1 multiples of 8 starting at 0; n: elements to add (multiple
// of 8, <= bounds[n_shards]); rank: this rank (it starts with its own shard).
int opk_clip_accumulate_group_push(const void* const* g, const float* const* scale, int n_group, float* const* acc_shards,
                                   const int64_t* bounds, int n_shards, int rank, int64_t n, void* stream);
// dst[0 .. nbytes) = src[0 .. nbytes) with this library's own copy kernel; either side may be peer-mapped memory of
// another GPU. Addresses and size are multiples of 16 bytes.
int opk_copy_bytes(void* dst, const void* src, int64_t nbytes, void* stream);

#ifdef __cplusplus
}
#endif
