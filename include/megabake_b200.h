/*
 * C ABI of the B200 decoder megakernel (libmegabake_b200.so).
 *
 * One handle owns the launch state for one decoder shape on one GPU.  Every
 * entry point returns an mk_error code, never throws, never allocates device
 * memory (the caller passes the workspace) and never synchronises unless its
 * comment says so.  Pointers are raw device addresses unless marked "host".
 * Streams are cudaStream_t passed as void*.
 *
 * Each entry point names the reference interface it stands in for, by path
 * inside the reference project.
 */
#ifndef MEGABAKE_B200_H
#define MEGABAKE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MK_MAX_LAYERS 96
#define MK_TOKEN_TILE 16

typedef enum mk_error {
  MK_OK = 0,
  MK_ERR_INVALID = 1,      /* bad argument (null, negative, inconsistent sizes)       */
  MK_ERR_UNSUPPORTED = 2,  /* shape outside what the kernel covers (see mk_last_error) */
  MK_ERR_CUDA = 3,         /* a CUDA runtime/driver call failed                         */
  MK_ERR_ALIGNMENT = 4,    /* a tensor base is not 16-byte aligned                      */
  MK_ERR_WORKSPACE = 5,    /* workspace too small                                       */
  MK_ERR_UNBOUND = 6,      /* launch before mk_bind_weights                             */
  MK_ERR_DEVICE_STATUS = 7 /* the device status word is not MK_STATUS_OK                */
} mk_error;

/* Device status word written by the kernel instead of trapping
 * (the reference traps: src/megabake/bodies/attention.py:540-543,
 *  src/megabake/bodies/generic.py:1159-1174). */
typedef enum mk_device_status {
  MK_STATUS_OK = 0,
  MK_STATUS_KV_OVERFLOW = 1, /* valid_length < 0 or valid_length + 1 > capacity */
  MK_STATUS_BAD_INDEX = 2,   /* token id or position out of range              */
  MK_STATUS_TIMEOUT = 3      /* a bounded device wait ran out                   */
} mk_device_status;

enum { MK_ROPE_HF = 0, MK_ROPE_HALF_SWAP = 1 };
/* TCGEN05: tensor-core projections (tcgen05.mma, TMEM accumulators) for every launch.
 * FMA: decode launches of at most 4 tokens run the small-launch kernel, which consumes its
 *      TMA-fed weight ring without tcgen05 (a matrix-vector product cannot fill a 128-row
 *      MMA): CUDA-core FMAs for one token (the row table: one grid barrier per launch),
 *      warp-level mma.sync for two to four; every other launch uses tcgen05.  Falls back to
 *      tcgen05 when the shape does not fit the small kernel (hidden > 2048 or a K slice
 *      longer than 2048).
 * AUTO: the faster of the two per launch; today the same choice as FMA.
 * (Value 1 named a bring-up engine without TMA or tensor cores; it is gone and rejected.)
 * Process-wide tunables of the small-launch kernel, read by mk_create: MEGABAKE_SMALL_RING_KB
 * (weight ring of the one-token kernel, 64..152, default 120) and MEGABAKE_SMALL_COPY_KB
 * (its largest weight copy, default 36). */
enum { MK_ENGINE_TCGEN05 = 0, MK_ENGINE_FMA = 2, MK_ENGINE_AUTO = 3 };

/* Decoder shape.  Mirrors the facts the reference reads off the captured graph
 * (src/megabake/lowering.py:1851-1870 for the attention contract,
 *  src/megabake/bodies/gemm.py:1887-1890 for the multiple-of-64 rule). */
typedef struct mk_config {
  int32_t hidden;
  int32_t layers;
  int32_t q_heads;
  int32_t kv_heads;
  int32_t head_dim;      /* 64 or 128 */
  int32_t intermediate;
  int32_t vocab;
  float rms_eps;
  int32_t qkv_bias;      /* 1: q/k/v projections carry a bias (addmm epilogue) */
  int32_t rope_style;    /* MK_ROPE_* */
  int32_t max_tokens;    /* largest batch (decode) or batch*sequence (prefill) per launch */
  int32_t max_positions; /* rows of the cos/sin tables */
  int32_t engine;        /* MK_ENGINE_* */
  int32_t sm_limit;      /* 0: one CTA per SM on the whole GPU; >0: use this many CTAs */
  /* Tensor parallel (0 or 1: off).  With tp_size > 1 this handle is one rank of a group on one
   * node: q_heads, kv_heads and intermediate are the rank's shard (q/k/v and gate/up sharded by
   * output rows, o and down by input columns), hidden is whole, vocab is the rows of this rank's
   * lm_head shard, embed_rows the rows of the (replicated) embedding table. */
  int32_t tp_size;
  int32_t tp_rank;
  int32_t embed_rows;    /* 0: same as vocab */
} mk_config;

typedef struct mk_layer_weights {
  const void* input_norm;  /* bf16 [hidden] */
  const void* q;           /* bf16 [q_heads*head_dim, hidden], row-major (nn.Linear.weight) */
  const void* k;           /* bf16 [kv_heads*head_dim, hidden] */
  const void* v;
  const void* q_bias;      /* bf16 [rows] or NULL */
  const void* k_bias;
  const void* v_bias;
  const void* o;           /* bf16 [hidden, q_heads*head_dim] */
  const void* post_norm;   /* bf16 [hidden] */
  const void* gate;        /* bf16 [intermediate, hidden] */
  const void* up;
  const void* down;        /* bf16 [hidden, intermediate] */
} mk_layer_weights;

typedef struct mk_weights {
  const void* embed;       /* bf16 [vocab, hidden] */
  const void* final_norm;  /* bf16 [hidden] */
  const void* lm_head;     /* bf16 [vocab, hidden]; equals embed when tied */
  const void* rope_cos;    /* bf16 [max_positions, head_dim] */
  const void* rope_sin;
  const mk_layer_weights* layers; /* host array of config.layers entries */
} mk_weights;

typedef struct mk_status_info {
  int32_t status;   /* mk_device_status */
  int32_t where;    /* kernel-internal wait/site id of the first failure */
  int32_t cta;
  int32_t detail;
} mk_status_info;

typedef struct mk_handle_s* mk_handle;

/* Bytes of device workspace mk_create needs for this shape on `device`.
 * Reference: the runtime-owned workspace of src/megabake/compiler.py:1979-1981. */
size_t mk_workspace_bytes(const mk_config* config, int device);

/* Create launch state.  `workspace` is device memory of at least
 * mk_workspace_bytes, 256-byte aligned, owned by the caller and kept alive
 * until mk_destroy; it is zeroed on `stream`.
 * Reference: compile_plan + _RuntimeState construction,
 * src/megabake/compiler.py:702-873, 1877-1981. */
int mk_create(const mk_config* config, void* workspace, size_t workspace_bytes, int device,
              void* stream, mk_handle* out);

/* Bind (or re-bind after the caller replaced a tensor) every parameter by
 * pointer; encodes the TMA descriptors and uploads the phase table on `stream`.
 * Reference: parameter rebinding in bind_callable / _fast_table_rebind,
 * src/megabake/compiler.py:980-997, 2216-2270, and build_table_descriptors,
 * src/megabake/bodies/gemm.py:1809-1843. */
int mk_bind_weights(mk_handle handle, const mk_weights* weights, void* stream);

/* One decode step for `batch` sequences, no sync: one cooperative launch (the small-launch kernel for
 * up to 4 sequences under MK_ENGINE_AUTO / MK_ENGINE_FMA when the shape allows, else the tensor engine).
 * ids/positions: int64 [batch].  key_caches/value_caches: host arrays of
 * config.layers device pointers, each bf16 [batch, capacity, kv_heads,
 * head_dim] contiguous.  valid_lengths: host array of config.layers device
 * pointers to int32 [1]; read, used as the append row, and advanced by one.
 * logits: bf16 [batch, vocab].
 * Reference: the bound callable's warm call, src/megabake/compiler.py:964-1081,
 * running the decode graph of tests/fixtures.py:247-312 whose attention is
 * megabake::kv_attention (src/megabake/lowering.py:211-247). */
int mk_decode(mk_handle handle, const int64_t* ids, const int64_t* positions, int batch,
              void* const* key_caches, void* const* value_caches, int32_t* const* valid_lengths,
              int capacity, void* logits, void* stream);

/* mk_decode for sequences of different lengths in one batch: valid_lengths[layer] points to int32 [batch],
 * one filled-position count per sequence (each is read, used as that sequence's append row and advanced by
 * one); sequence b attends over its own [0, valid_length[b]] and rotates with positions[b].  Everything else
 * as mk_decode.  Runs on the tensor engine (the context split follows the longest sequence; chunks past a
 * shorter sequence's end are empty).
 * Reference: none; its contract is one length shared by the batch (src/megabake/lowering.py:160-190,
 * README.md:29 lists per-sequence lengths as not supported). */
int mk_decode_ragged(mk_handle handle, const int64_t* ids, const int64_t* positions, int batch,
                     void* const* key_caches, void* const* value_caches, int32_t* const* valid_lengths,
                     int capacity, void* logits, void* stream);

/* `steps` greedy decode steps back to back without a host round trip: launch s picks each
 * sequence's token on the device (largest bf16 logit, lowest index among equal ones: what
 * torch.argmax returns), writes it to tokens_out[s * batch + b], stores it in ids[b] as the next
 * step's input and adds one to positions[b].  ids and positions (int64 [batch], device) are
 * therefore read and written; after the call they hold the inputs of the step that would come next.
 * logits: bf16 [batch, vocab], overwritten by every step (the last step's stay).  No sync.
 * A step whose prologue refuses (bad id/position, full cache) writes -1 tokens and NaN logits
 * and leaves ids, positions, caches and lengths alone; the status word says why.
 * Reference: none as an entry point; it stands in for the host loop of
 * benchmarks/full_model.py:277-335 (argmax on the host between two calls) and removes the
 * per-call host cost measured in ROADMAP.md:143. */
int mk_decode_steps(mk_handle handle, int64_t* ids, int64_t* positions, int batch, void* const* key_caches,
                    void* const* value_caches, int32_t* const* valid_lengths, int capacity, int steps,
                    int64_t* tokens_out, void* logits, void* stream);

/* One greedy decode step driven from host memory, in one call: copies `batch` ids and positions from
 * host_ids / host_positions (int64, pinned memory for the copies to be asynchronous) to the device,
 * runs the step with the device-side sampler, copies the sampled tokens to host_tokens_out and
 * SYNCHRONISES the stream before it returns.  Caches, lengths and logits as for mk_decode.  This is
 * the serving loop's step when the next id comes from the host (a scheduler, a stop criterion): three
 * small copies, one launch, one synchronisation, without the interpreter between them.
 * Reference: the host loop of benchmarks/full_model.py:277-335, one iteration. */
int mk_decode_step_host(mk_handle handle, const int64_t* host_ids, const int64_t* host_positions, int batch,
                        void* const* key_caches, void* const* value_caches, int32_t* const* valid_lengths,
                        int capacity, void* logits, int64_t* host_tokens_out, void* stream);

/* Stateless prompt pass over [batch, sequence] tokens with causal or additive
 * attention mask (bf16 [batch, 1, sequence, sequence], NULL = causal).
 * logits: bf16 [batch, sequence, vocab].
 * Reference: the mode="prefill" graph whose attention is megabake::attention
 * (src/megabake/lowering.py:273-300, src/megabake/fx_handler/hf_attention.py:28-61). */
int mk_prefill(mk_handle handle, const int64_t* ids, const int64_t* positions, const void* mask,
               int batch, int sequence, void* logits, void* stream);

/* y[M,N] = x[M,K] . W[N,K]^T (+ bias[N]), bf16 in/out, fp32 accumulate, one
 * rounding after the bias.  Runs the megakernel's projection engine on one
 * phase.  `handle` supplies workspace and engine; K a multiple of 64,
 * M <= config.max_tokens.  The two TMA descriptors are encoded on the host and travel in the
 * kernel's parameter block: no upload, no synchronisation.
 * Reference: the projection body, src/megabake/bodies/gemm.py:629-1114 with
 * its bias epilogue :1223-1251. */
int mk_linear(mk_handle handle, const void* x, const void* weight, const void* bias, void* y,
              int m, int n, int k, void* stream);

/* megabake::kv_attention on caller tensors (shapes as in mk_decode, one layer):
 * query bf16 [batch, 1, q_heads, head_dim], key/value bf16 [batch, 1, kv_heads,
 * head_dim] (already rotated), output bf16 [batch*q_heads, 1, head_dim].
 * Appends, attends, advances valid_length.
 * Reference: src/megabake/lowering.py:211-247. */
int mk_kv_attention(mk_handle handle, const void* query, const void* key, const void* value,
                    void* key_cache, void* value_cache, int32_t* valid_length, int batch,
                    int capacity, void* output, void* stream);

/* megabake::attention: query bf16 [batch, q_len, q_heads, head_dim], key/value
 * bf16 [batch, k_len, kv_heads, head_dim], mask bf16 additive [batch, 1, q_len,
 * k_len] or NULL, output bf16 [batch*q_heads, q_len, head_dim].
 * Reference: src/megabake/lowering.py:273-300. */
int mk_attention(mk_handle handle, const void* query, const void* key, const void* value,
                 const void* mask, float scale, int batch, int q_len, int k_len, void* output,
                 void* stream);

/* Synchronises `stream`, reads the device status word, and, if it is not OK,
 * resets the barrier/exchange counters so the handle can launch again.
 * Reference: none (the reference traps and loses the context). */
int mk_status(mk_handle handle, void* stream, mk_status_info* out);

/* Mirror of the device status word in host memory: `host_word` is one int32 of pinned, mapped host
 * memory (cudaHostAlloc / cudaHostRegister) that stays valid until it is replaced or the handle is
 * destroyed; NULL turns the mirror off.  A kernel that records a status other than OK also stores
 * it there, so the host can notice a refused or timed-out launch by reading the word, without a
 * synchronisation, before its next call.  mk_status clears the word when it resets the handle.
 * Reference: none (the reference traps; src/megabake/bodies/attention.py:540-543). */
int mk_set_status_mirror(mk_handle handle, int32_t* host_word);

/* Tensor-parallel decode (benchmark configuration "Llama-3-8B shape, heads and MLP columns sharded,
 * all-reduce after o_proj and down_proj").  The reference is single-device
 * (src/megabake/compiler.py:1518-1528 rejects inputs on more than one device), so these entry
 * points have no counterpart there.  Every rank is one process with one GPU and one handle created
 * with tp_size/tp_rank set.  Each rank owns an exchange buffer of mk_tp_exchange_bytes bytes
 * (256-byte aligned, plain cudaMalloc memory, zeroed) and makes it addressable by its peers
 * (mk_ipc_export / mk_ipc_open, or peer access inside one process); mk_tp_bind takes the tp_size
 * addresses, index = rank, as THIS process sees them.  After every rank has bound, the group
 * synchronises once on the host; from then on each mk_decode / mk_prefill call is made by all
 * ranks with the same batch and finishes its all-reduces inside the kernel: fp32 partial sums are
 * stored into every rank's buffer over NVLink, a stamped flag per source rank says they are there,
 * every wait is bounded (MK_STATUS_TIMEOUT names the rank that did not arrive), and each rank adds
 * the partial sums in rank order.  logits are this rank's vocabulary shard, bf16 [batch, vocab]. */
size_t mk_tp_exchange_bytes(const mk_config* config);
int mk_tp_bind(mk_handle handle, void* const* exchange, size_t exchange_bytes, void* stream);

/* A device allocation made addressable from another process on the same node (CUDA IPC):
 * export in the owner, open in the peer (peer access is enabled on first use), close when done.
 * `pointer` may lie inside a larger allocation: the offset travels with the handle. */
typedef struct mk_ipc_handle {
  unsigned char bytes[64];
  uint64_t offset;
} mk_ipc_handle;
int mk_ipc_export(void* pointer, mk_ipc_handle* out);
int mk_ipc_open(const mk_ipc_handle* in, void** pointer, void** base_out);
int mk_ipc_close(void* base);

/* Measurement baseline, outside the decoder path: y[M,N] = x[M,K] . W[N,K]^T (bf16, fp32 accumulate, no
 * bias) by the algorithm of the reference's only sm_100 kernel, its "blackwell_mma" body
 * (src/megabake/bodies/blackwell.py:91-159: 16 x 32 CTA tiles, four warps of mma.sync.m16n8k16,
 * per-element predicated global loads, no shared memory), restated in CUDA C.  The projection engine
 * (mk_linear) is timed against it by `python -m megabake_b200.bench_linear`. */
int mk_baseline_mma_gemm(const void* x, const void* weight, void* y, int m, int n, int k, void* stream);

/* Plain-text summary of what the handle will launch (CTAs, the form of the weight copies, tile height /
 * K split / chunks per copy / unit count of each projection phase per table).  Synchronous (reads the
 * phase tables back).  Reference: the plan report, src/megabake/plan.py:342-395. */
int mk_describe(mk_handle handle, char* buffer, size_t bytes);

/* Failure-detection hook for tests: adds `delta` to the grid-barrier count the host expects, so
 * that the next launch's first grid barrier can never be reached and its bounded wait
 * (MEGABAKE_WAIT_LIMIT_MS, read by mk_create; default 2000) runs out: the kernel records
 * MK_STATUS_TIMEOUT, raises the abort flag every other wait polls, and every CTA leaves through
 * the common exit.  mk_status then reports the timeout and resets the count.  Nothing waits
 * without a limit and nothing traps.
 * Reference: none (its barrier spins without a limit, src/megabake/runtime.py:157-159). */
int mk_debug_skew_barrier(mk_handle handle, uint32_t delta);

/* Event trace for the next launches: `buffer` is device memory of
 * ctas * events_per_cta * 8 bytes (NULL turns tracing off).  Worker thread 0 of
 * every CTA appends (event code << 56) | globaltimer-ns at phase entry, operand
 * staged, first accumulator ready, phase done, barrier passed, attention done;
 * a launch restarts each CTA's list at 0.
 * Reference: MEGABAKE_PHASE_TIMER stamps, src/megabake/runtime.py:27-46 and
 * src/megabake/codegen.py:1723-1751. */
int mk_set_trace(mk_handle handle, void* buffer, int events_per_cta);

/* Number of CTAs each launch uses, bytes of dynamic shared memory, kernels launched so far. */
int mk_launch_info(mk_handle handle, int32_t* ctas, int32_t* smem_bytes, int64_t* launches);

/* mk_kv_attention without a handle and without any device allocation, for callers
 * that may not allocate at the point of the call (a server that gave all of its HBM
 * to its own pool at start and forbids later allocations; a call site where an
 * allocation would serialise the device).  This entry point has no counterpart in
 * the reference.  The exchange buffers live in a 4 MiB array inside the library
 * image: batch * 16 * (192 * kv_heads + 4 * head_dim * q_heads) bytes (+ 512) must
 * fit, e.g. batch 16 x 32 heads x head_dim 64; larger shapes return
 * MK_ERR_WORKSPACE (use mk_kv_attention with a caller workspace).  `device` must be
 * the current device.  The first call on a device looks the array up, sets the
 * kernel attributes and clears the array on `stream`: make that call before any
 * stream capture begins.  All calls on a device share the one array: calls that
 * overlap (different streams or threads without ordering) race, so serialise
 * them.  The device status word is read (and cleared) by mk_kv_attention_static_status;
 * with valid_length == capacity the cache and the length are left untouched and the
 * output is filled with NaN, as with mk_kv_attention.  Tensors as in mk_kv_attention. */
int mk_kv_attention_static(int q_heads, int kv_heads, int head_dim, const void* query, const void* key,
                           const void* value, void* key_cache, void* value_cache, int32_t* valid_length,
                           int batch, int capacity, void* output, int device, void* stream);

/* Status word of the static scratch array on `device` (the current device): synchronises
 * `stream`, reports what the last mk_kv_attention_static launches recorded and, if that is not
 * MK_STATUS_OK (a full cache, a wait that ran out), clears the word and the abort flag and
 * restarts the barrier count, returning MK_ERR_DEVICE_STATUS.  Without this call a wait that
 * timed out once would leave the abort flag set in the array for the life of the process and
 * every later mk_kv_attention_static call on the device would leave at its first wait.
 * Allocates nothing.  No counterpart in the reference. */
int mk_kv_attention_static_status(int device, void* stream, mk_status_info* out);

/* Last error text for this thread (host string, valid until the next call). */
const char* mk_last_error(void);

int mk_destroy(mk_handle handle);

#ifdef __cplusplus
}
#endif
#endif /* MEGABAKE_B200_H */
