/*
 * b200_petals.h — C ABI of the sm_100a kernel library behind the pipeline stages.
 *
 * All entry points take raw device pointers and a CUDA stream (cudaStream_t cast
 * to void*), launch asynchronously on that stream, allocate nothing unless the
 * comment says so, and return 0 on success or a negative B200_E* code (the text
 * of the last error is available from b200_last_error()).
 *
 * Reference citations (jwkim-skku Mini-Petals, paths relative to the reference
 * root) name the torch op sequence each kernel replaces; the reference itself
 * contains no native code.
 */
#ifndef B200_PETALS_H_
#define B200_PETALS_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_OK 0
#define B200_EINVAL -1
#define B200_ECUDA -2
#define B200_ELIMIT -3

/* element types of activations / weights */
#define B200_F16 0
#define B200_BF16 1

const char* b200_last_error(void);
int b200_version(void);
/* Number of SMs of the current device (grid sizing for persistent kernels). */
int b200_sm_count(void);

/* ------------------------------------------------------------------ GEMM --
 * out[T,N] = epilogue( norm(x)[T,K] . W[N,K]^T )      (W = torch Linear weight)
 *
 * Swap-AB tcgen05 kernel: the weight is the 128-row M operand, streamed once
 * from HBM as pre-tiled, pre-swizzled 16 KiB blocks with bulk async copies;
 * tokens are the N operand (16..256 per tile), accumulators live in TMEM.
 * Work is split stream-K style over a persistent grid so that every SM streams
 * the same number of weight bytes whatever N and K are; partial tiles meet in
 * `scratch` and are summed in a fixed order (bit-reproducible).
 *
 * Opt-in fp8 weights (fp8 = 1): e4m3 weights with one scale per output row, activations quantised
 * per token on the fly, tcgen05.mma kind::f8f6f4, scales applied in the epilogue — half the weight
 * bytes per token (stands in for the reference's dead bitsandbytes NF4/INT8 path,
 * petals/server/server.py:88,189-191).
 *
 * Replaces q/k/v_proj, o_proj, gate/up/down_proj, lm_head and their
 * surrounding norm / activation / residual ops:
 * petals/llama/block.py:88-90,151,208-213,227-238; src/llama_partition.py:466-470.
 */
#define B200_EPI_NONE 0
#define B200_EPI_GELU_TANH 1 /* GPT-2 c_fc */
#define B200_EPI_SWIGLU 2    /* requires dual-packed gate/up weight */

#define B200_NORM_NONE 0
#define B200_NORM_RMS 1
#define B200_NORM_LAYER 2

/* Flag-chained decode step ("LL chain").  Between two kernel launches the GPU needs 3-4 us to notice that the
 * first grid is complete and to release the second one's dependency wait - five times per decoder block, with
 * the HBM idle.  With a chain the kernels of a decode step hand their activation vectors over as "LL words"
 * (two 16-bit values + a 32-bit tag in one 8-byte store, the scheme of the stream-K and tensor-parallel
 * exchanges): a consumer launched with programmatic stream serialization does NOT wait for the producer grid, it
 * polls the words it needs until they carry the tag (step number << 12 | id of the producing launch).  Words are
 * self-validating, so no fence, flag or grid dependency is needed, and a consumer starts on the first values while
 * the producer is still finishing others.  The caller numbers the producing launches of a step (ids 1..4095, unique
 * within the step), advances *seq once per step BEFORE the step's first launch (stream order), launches every kernel
 * of the step with pdl = 1 into one stream, and ends the step with an ordinary (grid-dependent) kernel.
 * LL buffers: [T][ld] 8-byte words, word i of a row = elements 2i, 2i+1; zero-initialised once.
 * Replaces nothing in the reference (its blocks are eager torch ops, petals/llama/block.py:200-240); it removes the
 * launch-boundary cost that CUDA graphs alone (petals/llama/cuda_graphs.py) leave in place. */
typedef struct b200_ll_chain {
    const int32_t* seq;   /* device: the step number (> 0); NULL = chain off, everything below ignored */
    const void* x_ll;     /* input vector as LL words (the kernel then never reads args->x) */
    const void* res_ll;   /* residual as LL words, when args->residual is set */
    void* out_ll;         /* output as LL words (16-bit outputs; args->out is still written when non-NULL) */
    int32_t ldx_ll, ldr_ll, ldo_ll;   /* row strides in words */
    int32_t x_op, res_op, out_op;     /* launch ids: who produced x / the residual, and this launch's own id */
    int32_t half;         /* 0/1: half of ll_buf for this launch's stream-K exchange; alternate between consecutive GEMMs */
    int32_t reserved;
} b200_ll_chain;

typedef struct b200_gemm_args {
    const void* w_packed; /* b200_pack layout, see ops/packing.py */
    const void* x;        /* [T, K] 16-bit, row stride ldx elements */
    void* out;            /* [T, N] 16-bit (or fp32 when out_fp32), row stride ldo */
    const void* residual; /* [T, N] 16-bit added after the epilogue, or NULL */
    const void* bias;     /* [N] 16-bit, or NULL */
    const void* norm_w;   /* [K] 16-bit norm gain (norm_mode != 0) */
    const void* norm_b;   /* [K] 16-bit LayerNorm beta, or NULL */
    float* scratch;       /* >= b200_gemm_scratch_bytes() bytes */
    int32_t* counters;    /* >= n_tiles * t_tiles ints, all zero; left all zero */
    int32_t T, N, K;      /* logical sizes; K is the packed (64-padded) K */
    int32_t ldx, ldo, ldr;
    int32_t n_tiles;      /* packed 128-row tiles (dual: pairs) */
    int32_t dual;         /* 1 = gate/up interleaved per tile */
    int32_t epilogue;
    int32_t norm_mode;
    float norm_eps;
    int32_t dtype;        /* B200_F16 / B200_BF16 */
    int32_t out_fp32;
    int32_t grid;         /* 0 = one CTA per SM */
    int32_t pdl;          /* 1 = launch with programmatic stream serialization */
    int32_t debug;        /* 0 in production; experiment switches, see csrc/gemm.cu */
    int32_t fp8;          /* 1 = e4m3 weights with one scale per output row (pack_weight_fp8, needs w_scale);
                             2 = OCP-MX: e4m3 weights with one UE8M0 scale per 32 elements along k packed behind every
                             k-block (pack_weight_mx), activations block-quantised on the fly,
                             tcgen05.mma.kind::mxf8f6f4.block_scale with the scales in tensor memory.  T <= 32, K % 128 == 0 */
    const float* w_scale; /* fp8: per-output-row dequantisation scale, [n_tiles*128] (dual: gate rows then up rows) */
    /* Optional L2 warm-up for the kernels that follow in the stream (b200_gemm only): once a CTA has issued
     * its last weight load it asks the L2 for its share of up to two byte ranges (cp.async.bulk.prefetch.L2),
     * typically the head of the next linear's packed weights, so the HBM keeps streaming through this
     * kernel's fix-up / epilogue and the next kernel's launch.  NULL / 0 = none.  Ranges must be 16-byte
     * aligned device memory that stays valid until the stream has passed this kernel. */
    const void* prefetch[2];
    int64_t prefetch_bytes[2];
    /* Optional ticket-free fix-up for decode sizes (b200_gemm with T <= 16; b200_gemm_allreduce / b200_gemm_gather and
     * fp8 weights with T <= 4):
     * b200_gemm_ll_bytes() bytes of device memory, zeroed ONCE by the caller and then owned by the library
     * (one buffer per stream of GEMM launches; it may be shared by all GEMMs of that stream).  When every
     * output tile is split over the same whole number of CTAs, the CTAs publish their partial sums as
     * (value, tag) 8-byte words and the tile's last CTA polls for them and clears them again - no fence, no
     * atomic ticket, no counter (3-way split: 2.3 -> 0.4 us, 8-way: 5.9 -> 1.6 us per launch at T = 1; with 2..16 tokens every CTA of the
     * tile reduces a share of its elements).  Same summation
     * order as the ticket path, i.e. bit-identical results.  NULL = ticket path. */
    void* ll_buf;
    /* Optional with norm_mode == B200_NORM_RMS: per-token 1/rms computed beforehand (b200_rms_rstd, same bits as the
     * in-kernel statistics); the kernel then skips its own statistics pass.  Pays off from ~8 tokens per step. */
    const float* rstd;
    /* Optional flag chain (decode sizes, 16-bit weights, b200_gemm only): see b200_ll_chain. */
    b200_ll_chain chain;
} b200_gemm_args;

int b200_gemm(const b200_gemm_args* args, void* stream);
/* Upper bound of the scratch needed by any b200_gemm call with T <= max_tokens. */
int64_t b200_gemm_scratch_bytes(int32_t max_tokens);
int64_t b200_gemm_ll_bytes(void);
/* Token-tile width the kernel will pick for T tokens (16,32,64,128,256). */
int32_t b200_gemm_token_tile(int32_t T, int32_t dual);

/* Prefill-size variant (T >= 64, no norm prologue, 16-bit weights; same argument struct, scratch and
 * counters unused): weights by cp.async.bulk, activations by a 2-D TMA tensor map, two TMEM accumulator
 * buffers so the epilogue of a tile overlaps the main loop of the next. */
int b200_gemm_prefill(const b200_gemm_args* args, void* stream);

/* Row-parallel linear of a tensor-parallel span with the all-reduce fused into the tile epilogue
 * (decode sizes, T <= 16): every rank runs this with its K shard of the weight; the CTA that finishes
 * an output tile pushes its fp32 partial into every rank's staging buffer with peer stores over
 * NVLink, waits for the other ranks' partials of the same tile (flags in local memory), adds them in
 * rank order and applies bias / residual once.  All ranks end with bit-identical outputs; tiles are
 * exchanged while other tiles are still in the tensor core.  The reference's dead TP path runs an
 * NCCL all-reduce after each row-parallel linear (petals/server/backend.py:134-136 via tensor_parallel).
 * stage[r] / flags[r] are rank r's buffers mapped into this process (e.g. torch symmetric memory):
 *   stage: 2 * world * 16 * n_max floats,  flags: 2 * world * tiles_max ints (zeroed once),
 *   seq / exit_counter: one int each, local, zeroed once.  All ranks must issue the same sequence of
 *   b200_gemm_allreduce calls on a workspace. */
typedef struct b200_tp_args {
    int32_t world, rank, n_max, tiles_max;
    void* stage[8];
    void* flags[8];
    int32_t* seq;
    int32_t* exit_counter;
    int32_t mode;   /* 0: the producer waits and reduces (all-reduce in one kernel); 1: the producer only pushes
                       its partial tiles and the next GEMM (b200_gemm_gather) waits for them and adds them up */
} b200_tp_args;
int b200_gemm_allreduce(const b200_gemm_args* args, const b200_tp_args* tp, void* stream);
/* Consumer of a mode-1 producer ("all-gather -> GEMM"): every CTA first rebuilds
 * x[t,:] = residual[t,:] + bias + sum over ranks of the pushed partial rows (rank order, bit-identical on
 * all ranks), stores it to args->x, then runs b200_gemm on it.  The NVLink latency of the exchange hides
 * behind the launch of this kernel instead of sitting at the producer's tail. */
int b200_gemm_gather(const b200_gemm_args* args, const b200_tp_args* tp, const void* residual, int32_t ldr,
                     const void* bias, void* stream);

/* Row-parallel linear of a tensor-parallel span at PREFILL sizes: all-reduce of the ranks' partial outputs through
 * the NVSwitch (NVLS) with the linear's epilogue in the same kernel: out = sum_r partial_r + bias + residual on every
 * rank.  Each rank reads its slice of the elements through the multicast address with multimem.ld_reduce (the switch
 * adds the ranks' values, fp32 accumulation), applies bias / residual, and writes the slice through the multicast
 * address of the output with multimem.st (replicated into every rank's memory): reduce-scatter by load, all-gather by
 * store, no rank polls its peers in turn.  The reference's dead TP path: NCCL all-reduce + separate torch adds
 * (petals/server/backend.py:134-136).
 *   mc_partial / mc_out  MULTICAST addresses (e.g. torch symmetric memory, handle.multicast_ptr + offset) of two
 *                        symmetric buffers; every rank's GEMM wrote its [T, N] partial into its own copy of the first.
 *   flags_local / flags_peer[r]  16 ints of symmetric memory per rank (zeroed once): this rank's copy and every rank's.
 *   seq, cta_done        one int each, local, zeroed once.  All ranks must issue the same sequence of calls. */
typedef struct b200_nvls_args {
    const void* mc_partial;
    void* mc_out;
    const void* residual;  /* local [T, ldr] 16-bit, or NULL */
    const void* bias;      /* [N] 16-bit, or NULL */
    int32_t T, N, ldp, ldo, ldr, dtype;
    int32_t world, rank;
    int32_t* flags_local;
    void* flags_peer[8];
    int32_t* seq;
    int32_t* cta_done;
    int32_t pdl, reserved;
} b200_nvls_args;
int b200_tp_allreduce_nvls(const b200_nvls_args* args, void* stream);

/* b200_gemm for callers that cannot allocate device memory (no counterpart in the reference, which
 * has no native code and lets torch allocate freely).  Same arguments and result as b200_gemm, but
 * args->scratch and args->counters are ignored: the workspace is a fixed ~5 MiB array inside the
 * library image, resolved per device on the first call made on that device (make that call before
 * starting a stream capture).  Limits: T <= 16 tokens, <= 2048 output tiles, <= 160 CTAs; beyond
 * them the call returns B200_ELIMIT.  Calls share the one array: keep them on one stream — kernels
 * from two calls that overlap on the GPU race on it.  args->pdl and args->ll_buf are ignored.
 * Performs no cudaMalloc/cudaFree. */
#define B200_GEMM_STATIC_MAX_TOKENS 16
int b200_gemm_static_scratch(const b200_gemm_args* args, void* stream);

/* ------------------------------------------------------------- attention --
 * Decode: for each of T independent sessions' new tokens, apply RoPE to q and k,
 * append k/v to that session's pre-allocated cache in place (no torch.cat
 * reallocation as in petals/llama/block.py:123-128), and attend over the cache
 * with a split-KV online softmax (GQA heads of one kv head share the K/V
 * stream; no repeat_kv copy, block.py:131-132).  Scores never touch HBM
 * (block.py:134-141 materialises [nh,T,S] in fp32).
 * kv_ptrs[t] = {K base, V base} of this layer for token t's session, each
 * laid out [n_kv_heads][s_max][head_dim]; pos[t] = tokens already cached.
 */
typedef struct b200_attn_decode_args {
    const void* qkv;        /* [T, (nh + 2 nkv) * d] : q | k | v, row stride ldqkv */
    void* out;              /* [T, nh * d], row stride ldo */
    const uint64_t* kv_ptrs;/* device [T][2] */
    const int32_t* pos;     /* device [T] */
    const float* inv_freq;  /* device [d/2] RoPE inverse frequencies, NULL = no RoPE (GPT-2) */
    float* scratch;         /* >= b200_attn_decode_scratch_bytes() */
    int32_t* counters;      /* T * n_kv_heads ints, zero on entry and on exit */
    int32_t T, n_heads, n_kv_heads, head_dim, s_max, splits, ldqkv, ldo;
    float scale;            /* 1/sqrt(d) */
    int32_t dtype, pdl;
    /* Optional: 2 * b200_attn_decode_scratch_bytes() bytes, zeroed ONCE by the caller, then owned by the library
     * (one per stream).  The KV splits of a head then publish their partial (o, m, l) as (value, tag) 8-byte
     * words and the last split polls, merges and clears them: no fence / atomic ticket in the merge.  Same
     * arithmetic and order as the ticket path.  NULL = ticket path (scratch + counters). */
    void* ll_scratch;
    /* Optional flag chain (see b200_ll_chain): qkv is read from chain.x_ll (tag of chain.x_op) instead of waiting for
     * the producer grid, the output also goes to chain.out_ll with chain.out_op; needs ll_scratch.  res_* unused. */
    b200_ll_chain chain;
} b200_attn_decode_args;
int b200_attn_decode(const b200_attn_decode_args* args, void* stream);
int64_t b200_attn_decode_scratch_bytes(int32_t T, int32_t n_heads, int32_t head_dim, int32_t splits);

/* Prefill / chunk: rotate q in place, rotate k and store k, v into the session cache at
 * positions [pos0, pos0 + T).  (HF rotary + cache append, block.py:96-128.) */
int b200_rope_append(void* qkv, void* kcache, void* vcache, const float* inv_freq, int32_t T, int32_t n_heads,
                     int32_t n_kv_heads, int32_t head_dim, int32_t s_max, int32_t ldqkv, int32_t pos0,
                     int32_t dtype, int32_t pdl, void* stream);
/* Causal attention of a T-token chunk (already appended) against cache rows [0, pos0 + T).
 * The reference never builds the causal mask on its live path; this does. */
int b200_attn_prefill(const void* q, void* out, const void* kcache, const void* vcache, int32_t T, int32_t n_heads,
                      int32_t n_kv_heads, int32_t head_dim, int32_t s_max, int32_t ldq, int32_t ldo, int32_t pos0,
                      float scale, int32_t dtype, int32_t pdl, void* stream);

/* Same contract on the tensor cores: 128-query x 128-key tiles, S = QK^T and O = PV by tcgen05.mma
 * (V consumed in place as an MN-major operand), online softmax between them, accumulators in TMEM. */
int b200_attn_prefill_tc(const void* q, void* out, const void* kcache, const void* vcache, int32_t T, int32_t n_heads,
                         int32_t n_kv_heads, int32_t head_dim, int32_t s_max, int32_t ldq, int32_t ldo, int32_t pos0,
                         float scale, int32_t dtype, int32_t pdl, void* stream);
/* The same kernel over cache planes with any element strides between positions (pos_stride) and between kv heads
 * (head_stride), e.g. planes that keep all heads of a position side by side: pos_stride = row, head_stride = head_dim.
 * Strides and addresses must be multiples of 16 bytes. */
int b200_attn_prefill_tc_rows(const void* q, void* out, const void* kcache, const void* vcache, int32_t T, int32_t n_heads,
                              int32_t n_kv_heads, int32_t head_dim, int32_t s_max, int32_t ldq, int32_t ldo, int32_t pos0,
                              float scale, int32_t dtype, int64_t pos_stride, int64_t head_stride, int32_t pdl, void* stream);

/* ----------------------------------------------------------- elementwise --
 * Embedding gather (+ learned positions for GPT-2): src/llama_partition.py:107.
 * ids are int64 on the device (the last stage writes them there). */
int b200_embed(const void* ids, const void* pos, int32_t pos0, const void* wte, const void* wpe, void* out, int32_t T,
               int32_t H, int32_t vocab, int32_t max_pos, int32_t dtype, int32_t pdl, void* stream);
/* Head of a flag chain: the 16-bit rows x[T, H] (already complete in stream order) re-published as LL words tagged
 * (*seq << 12 | op), so that the chain's first GEMM can poll them like any other link of the chain. */
int b200_ll_publish(const void* x, int32_t ldx, void* out_ll, int32_t ld_ll, int32_t T, int32_t H, const int32_t* seq,
                    int32_t op, int32_t pdl, void* stream);
/* Standalone RMSNorm (layer_norm=0) / LayerNorm (1) for prefill-size inputs: block.py:208-213. */
/* rstd[t] = 1/sqrt(mean(x[t]^2) + eps), one block per token; see b200_gemm_args.rstd. */
int b200_rms_rstd(const void* x, float* rstd, int32_t T, int32_t K, int32_t ldx, float eps, int32_t dtype, int32_t pdl,
                  void* stream);
int b200_norm(const void* x, const void* w, const void* b, void* out, int32_t T, int32_t H, int32_t ldx, int32_t ldo,
              float eps, int32_t layer_norm, int32_t dtype, int32_t pdl, void* stream);
/* Greedy sampling: first index of the row maximum of fp32 logits (src/rpc_handler.py:331-335).
 * part_val/part_idx: T*chunks scratch; counters: T ints kept zero. */
int b200_argmax(const float* logits, int32_t ld, int32_t T, int32_t V, float* part_val, int32_t* part_idx,
                int32_t* counters, void* out_ids, int32_t chunks, int32_t pdl, void* stream);

/* Arg-max over one SHARD of the vocabulary (vocab-sharded LM head): indices are reported with `idx_offset` added,
 * `init_pair` (T x {float bits, int32 index}, or NULL) is a candidate from another shard that the shard's own
 * maximum has to beat (ties go to the lower index, as torch.argmax would on the whole row), and `out_pair`
 * (T x 2 words, or NULL) receives the winning (value, index) so that the next shard can continue.  out_ids may be NULL. */
int b200_argmax_partial(const float* logits, int32_t ld, int32_t T, int32_t V, float* part_val, int32_t* part_idx,
                        int32_t* counters, void* out_ids, int32_t chunks, int32_t idx_offset, const void* init_pair,
                        void* out_pair, int32_t pdl, void* stream);

/* ---------------------------------------------------------- pipeline hop --
 * Hidden-state handoff between two pipeline stages on different GPUs of one NVSwitch box, made of two small
 * kernels that are captured into the stages' CUDA graphs: b200_hop_send (last node of the producer's graph) writes
 * the micro-batch into a ring in the RECEIVER's memory with peer stores over NVLink, each 4-byte payload paired
 * with the message number in one 8-byte word; b200_hop_recv (first node of the consumer's graph) polls its own
 * memory until the whole message carries the expected number and unpacks it.  No host, no flag, no fence, no
 * library call on the per-token path.  Replaces the reference's hop through the client:
 * src/rpc_transport.py:736-766 (GPU -> CPU -> serialize -> libp2p -> deserialize -> GPU, twice per stage).
 *   ring     b200_hop_ring_bytes(depth, t_max, pairs_per_token) bytes in the receiver's memory, zeroed once; the
 *            sender passes the peer-mapped address (e.g. torch symmetric memory), the receiver its local one.
 *            Message n uses entry n % depth: depth must exceed the number of messages the link can have in flight.
 *   counter  one int per link END (sender and receiver each own one, both start at 0, local memory).
 *   x        [T, hidden] 16-bit rows (send: source, recv: destination), row stride ldx elements; hidden may be 0.
 *   extra    [T, n_extra] 32-bit words that travel with each token (token ids, arg-max partials), or NULL.
 * A receive that sees nothing for timeout_ms (0 = 30 s) prints a message and traps instead of hanging the GPU. */
typedef struct b200_hop_args {
    void* x;
    void* extra;
    void* ring;
    int32_t* counter;
    int32_t T, hidden, ldx, n_extra;
    int32_t depth, t_max, pairs_per_token;
    int32_t timeout_ms, pdl;
} b200_hop_args;
int64_t b200_hop_ring_bytes(int32_t depth, int32_t t_max, int32_t pairs_per_token);
int b200_hop_send(const b200_hop_args* args, void* stream);
int b200_hop_recv(const b200_hop_args* args, void* stream);
/* Loads the two kernels on the current device (call once before capturing them into a graph). */
int b200_hop_init(void);

/* Opt-in device-side event trace of the decode kernels (profiling aid, scripts/trace_decode.py): the GEMM and the
 * decode attention stamp %globaltimer at entry / after their dependency wait / first accumulator / exit for the first
 * and last CTA.  buf: 8 * (1 + 2 * cap) bytes of zeroed device memory ([0] = events written, then (ns, tag) pairs with
 * tag = kernel << 56 | aux << 32 | phase << 16 | last_cta; aux of a GEMM = n_tiles | k_blocks << 12); NULL = off.  Synchronous (cudaMemcpyToSymbol); the reference's only
 * timing aid is time.time() around forward calls (src/rpc_handler.py:190-249). */
int b200_trace_set(void* buf, int32_t cap);

/* Temperature / top-k / top-p / repetition-penalty sampling on the device with the reference's rules
 * (src/rpc_handler.py:327-403), one CTA per row, no sort (radix descent over float bit patterns).
 * rows: T records {float temperature, top_p, penalty; int32 top_k, n_recent; int32 recent[50]} on the
 * device (b200_sample_row_bytes() each); uniforms: T floats in [0,1) (e.g. torch.rand on the device,
 * philox); probs: T*V floats of scratch, holds the final un-normalised distribution on return. */
int32_t b200_sample_row_bytes(void);
int b200_sample(const float* logits, int32_t ld, int32_t T, int32_t V, const void* rows, const float* uniforms,
                float* probs, void* out_ids, int32_t pdl, void* stream);
/* The same with the sessions' sampling state on the device: rows[row_index[t]] (row_index NULL: rows[t]) holds the
 * parameters and the window of recent tokens, states[..] = {uint64 seed, uint64 draws so far}
 * (b200_sample_state_bytes() each).  The uniform number of a draw is the first word of
 * Philox4x32-10(key = seed, counter = draws so far); after the draw the kernel appends the token to the window and
 * advances the stream.  Nothing comes from the host per step, so the call can sit in a captured graph, and a session's
 * tokens depend only on its seed (the reference draws from torch's global generator on whichever server samples,
 * src/rpc_handler.py:396-403). */
int32_t b200_sample_state_bytes(void);
int b200_sample_stateful(const float* logits, int32_t ld, int32_t T, int32_t V, void* rows, void* states,
                         const int32_t* row_index, float* probs, void* out_ids, int32_t pdl, void* stream);


/* =====================================================================================================
 * Mechanisms for layer-list decoder designs with an fp32 residual stream (first user: Gigezen).
 * Activations that enter a tensor-core GEMM are 16-bit; the residual stream, norms, rotary angles,
 * attention scores and weights, and routers are fp32.  Element type codes: B200_F16 / B200_BF16 / B200_F32.
 * The reference has no counterpart (its blocks are HF Llama layers, petals/llama/block.py).
 * ===================================================================================================== */
#define B200_F32 2

/* out[t, :] = table[ids[t], :] as fp32 (table 16-bit or fp32); ids int64 on the device. */
int b200_embed_f32(const void* ids, const void* table, int32_t table_dtype, float* out, int32_t T, int32_t width,
                   int32_t ldo, int32_t vocab, int32_t pdl, void* stream);

/* Residual update + RMS norm in one pass over the fp32 stream, one block per token:
 *     x[t] += add_a[t] + add_b[t] + sum_k pair_w[t*top+k] * pair_y[t*top+k]        (each term optional)
 *     out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * (gain_offset + gain)               (out optional)
 * gain is fp32; gain_offset = 1 for gains stored around zero, 0 for plain gains.  out: 16-bit or fp32, row stride ldo
 * (columns beyond width are not touched).  The k-sum runs in index order (bit-reproducible). */
typedef struct b200_add_norm_args {
    float* x;
    const float* add_a;
    const float* add_b;
    const float* pair_y;
    const float* pair_w;
    const float* gain;
    void* out;
    int32_t T, width, ldx, lda, ldb, ldp, top, ldo, out_dtype;
    float eps, gain_offset;
    int32_t pdl;
    float add_scale;      /* x += add_scale * (add_a + add_b + pairs); a residual multiplier (1 = plain sum) */
} b200_add_norm_args;
int b200_add_rms_norm(const b200_add_norm_args* args, void* stream);

/* Gated unit with clamps: g = min(gate, limit), u = clamp(up, -limit, limit), act = g * sigmoid(alpha * g) * (u + up_shift).
 * gate/up: fp32 [T, ff] each (row stride ld); act: 16-bit or fp32 [T, ff] (row stride ldo).  limit <= 0: no clamps. */
int b200_glu_clamp(const float* gate, const float* up, int32_t ld, void* act, int32_t ldo, int32_t out_dtype, int32_t T,
                   int32_t ff, float limit, float alpha, float up_shift, int32_t pdl, void* stream);

/* Plain fp32-accumulating GEMM on the CUDA cores: out[r, n] = sum_k x[src(r), k] * w[g(r)][n, k].
 * True 32-bit products (fmaf), used where the tensor-core GEMM's 16-bit operands are not allowed (the all-fp32 mode)
 * and for the small batched / grouped products around latent attention and the experts of a mixture.
 *   batch > 1: independent problems b = 0..batch-1 at x + b*x_bs, w + b*w_bs, out + b*o_bs (element strides).
 *   group_off != NULL: rows [group_off[g], group_off[g+1]) use weight w + g*w_gs (device table, groups + 1 ints);
 *                      T is then an upper bound of group_off[groups].
 *   row_src / row_dst: optional gather of x rows / scatter of out rows (ints per problem row).
 *   w2 != NULL: out = silu(x.w^T) * (x.w2^T)   (gate / up of an expert).
 *   row_scale: optional factor per problem row, applied last. */
typedef struct b200_simt_gemm_args {
    const void* x;
    const void* w;
    const void* w2;
    void* out;
    const int32_t* row_src;
    const int32_t* row_dst;
    const int32_t* group_off;
    const float* row_scale;
    int32_t T, N, K, ldx, ldw, ldo;
    int32_t x_dtype, w_dtype, out_dtype;
    int32_t batch, groups;
    int64_t x_bs, w_bs, o_bs, w_gs;
    int32_t pdl, reserved;
} b200_simt_gemm_args;
int b200_gemm_simt(const b200_simt_gemm_args* args, void* stream);

/* Latent attention, step 1: rotary positions and cache append, one block per token.
 *   proj[t]: fp32 row holding q (heads x [dim unrotated | rot rotated]) at column q_off and, at kv_off (< 0: this
 *   layer reads another layer's cache and writes nothing), [kv_rank latent | rot shared rotated key].
 *   q's rotated parts are rotated in place.  The latent is RMS-normed (plain gain, fp32) and stored with the rotated
 *   key part as one cache row [kv_rank + rot] (16-bit or fp32) at the token's position.
 *   Rotation: the first rot_dims of the rot part, pairs (i, i + rot_dims/2), angle = pos * inv_freq[i] evaluated in
 *   double precision (inv_freq: double [rot_dims/2]).
 *   Cache row of token t: kv_ptrs ? kv_ptrs[t * kv_ptr_stride] + pos[t] * row_bytes : cache + (pos0 + t) * row_bytes. */
typedef struct b200_latent_args {
    float* proj;
    int32_t ldp, q_off, kv_off;
    const float* c_gain;
    const double* inv_freq;
    void* cache;
    const uint64_t* kv_ptrs;
    const int32_t* pos;
    int32_t kv_ptr_stride, pos0;
    int32_t T, heads, dim, rot, rot_dims, kv_rank, row_elems, cache_dtype;
    float eps;
    /* step 2 (b200_latent_attn) */
    const float* q_abs;   /* [T, heads, kv_rank] fp32: unrotated query pulled through the key up-projection */
    float* out;           /* [T, heads, kv_rank] fp32: softmax-weighted sum of latents */
    int32_t ldqa, ldout, window;
    float scale;
    int32_t pdl, reserved;
} b200_latent_args;
int b200_latent_rope_append(const b200_latent_args* args, void* stream);
/* Step 2: for the token at position pos, the keys are the cached rows j in (pos - window, pos]; score
 * s(j) = (q_abs . c_j + q_rot . kr_j) * scale, softmax in fp32, out = sum_j p_j c_j.  All heads of a token share the cached rows (one block = one token x 8 heads,
 * keys staged through shared memory 32 at a time). */
int b200_latent_attn(const b200_latent_args* args, void* stream);
/* The same with the window's keys of every token divided over `splits` blocks (decode sizes, where tokens x heads alone
 * do not fill the GPU); the shares meet in `scratch` (b200_latent_attn_scratch_bytes) and are merged in index order by a
 * second launch.  splits = 1 is b200_latent_attn. */
int b200_latent_attn_split(const b200_latent_args* args, int32_t splits, float* scratch, void* stream);
int64_t b200_latent_attn_scratch_bytes(int32_t T, int32_t heads, int32_t kv_rank, int32_t splits);

/* Latent attention of a prompt-size chunk of ONE session on the tensor cores (16-bit modes).  The visible latents are
 * expanded beforehand by a GEMM into per-head keys and values, kvx[r] = [W_uk c | W_uv c] of key position s0 + r
 * (unrotated keys of head h at column h * dim, values at v_off + h * vdim; s0 <= first visible key of the chunk);
 * the rotated key part is read from the session's cache rows (column kv_rank).  proj holds the chunk's queries (fp32,
 * rotated part already rotated, see b200_latent_rope_append).  Sliding-window flash attention with mma.sync m16n8k16:
 * scores and softmax in fp32, the weights enter P.V as two 16-bit terms (hi + lo).  out: 16-bit [T, heads * vdim]. */
int b200_latent_attn_prefill(const float* proj, int32_t ldp, int32_t q_off, const void* kvx, int32_t ldkv, int32_t v_off,
                             const void* cache, int32_t row_elems, int32_t kv_rank, void* out, int32_t ldo, int32_t T,
                             int32_t heads, int32_t dim, int32_t rot, int32_t vdim, int32_t pos0, int32_t s0, int32_t window,
                             float scale, int32_t dtype, int32_t pdl, void* stream);

/* Router of a mixture of experts, one warp per token.  s = softmax(logits) over all `experts` (fp32).  Group-limited
 * top-k: consecutive experts are partitioned into `groups` blocks, a block is ranked by max(s) inside it, and the
 * candidates are the members of the `keep` highest-ranked blocks; among the candidates the `top` highest s are taken
 * (lowest index on ties).  ids [T, top] int32; weights [T, top] fp32 = s of the taken experts as it is
 * (renorm != 0: divided by their sum). */
int b200_moe_route(const float* logits, int32_t ld, int32_t T, int32_t experts, int32_t groups, int32_t keep, int32_t top,
                   int32_t renorm, int32_t* ids, float* weights, int32_t pdl, void* stream);
/* Sorts the T*top (token, slot) pairs by expert (single block): group_off [experts + 1], row_pair [T*top] (pair
 * index t*top+k per sorted row) and row_token [T*top] (t per sorted row). */
/* Dense form of the experts for tensor-core GEMMs: after ONE gate/up GEMM over all experts' concatenated rows
 * (act [T, experts * ff], 16-bit), every token's slice of expert e is multiplied by that expert's routing weight
 * (0 when it was not chosen), so that ONE down GEMM over the concatenated experts yields the weighted sum. */
int b200_moe_scale(void* act, int32_t ld, int32_t dtype, const int32_t* ids, const float* weights, int32_t T,
                   int32_t experts, int32_t ff, int32_t top, int32_t pdl, void* stream);
int b200_moe_plan(const int32_t* ids, int32_t T, int32_t top, int32_t experts, int32_t* group_off, int32_t* row_pair,
                  int32_t* row_token, int32_t pdl, void* stream);

/* Embedding gather to fp32 with a learned position vector added: out[t] = table[ids[t]] + pos_table[p_t],
 * p_t = pos ? pos[t] : pos0 + t (clamped to the table). */
int b200_embed_pos_f32(const void* ids, const void* table, const void* pos_table, int32_t table_dtype, const int32_t* pos,
                       int32_t pos0, float* out, int32_t T, int32_t width, int32_t ldo, int32_t vocab, int32_t max_pos,
                       int32_t pdl, void* stream);

/* Piecewise activation of a feed-forward layer with two learned numbers (a_pos, a_neg: device floats at `params`):
 *   z > 0:  softplus(a_pos) z^2 + lin z;     z <= 0:  (neg_base + softplus(a_neg)) (exp(z) - 1 - z) + lin z.
 * z: fp32 [T, ff] (row stride ld); act: 16-bit or fp32 [T, ff] (row stride ldo). */
int b200_xielu(const float* z, int32_t ld, const float* params, float lin, float neg_base, void* act, int32_t ldo,
               int32_t out_dtype, int32_t T, int32_t ff, int32_t pdl, void* stream);

/* Grouped-query softmax attention without rotation, with a sink in the denominator.
 * proj[t] (fp32 row of the fused projection): q [heads x dim] at q_off, k [kv_heads x dim] at k_off, v [kv_heads x vdim] at
 * v_off, one gate logit per head at g_off.
 * Step 1, b200_sink_attn_append (three blocks per token): adds `bias` (q | k | v order, may be NULL); RMS-norms the WHOLE q
 * row and the WHOLE k row (gains q_gain / k_gain, eps); folds scale * temp[h] into q (written back in place); divides every
 * value head by its root mean square over vdim (eps, no gain); vmix_mode 1: leaves the values in v_first[t]; 2: v <- (1 - l)
 * v + l v_first[t] with l = *vmix; then stores k and v as rows of the key / value planes at the token's position.
 * Planes: one row [row_elems] per position, heads side by side; of token t: kv_ptrs ? kv_ptrs[t * kv_ptr_stride + {0, 1}]
 * : k_cache / v_cache; position pos ? pos[t] : pos0 + t.
 * Step 2, b200_sink_attn (one block per token, head and share): s_j = q . k_j for j <= position, weights
 * exp(s_j) / (sink + sum_i exp(s_i)) (sink = 1: one more key of score 0 and no value; 0: plain softmax), fp32 throughout;
 * out[t, h] = sigmoid(gate logit) * sum_j w_j v_j (16-bit or fp32, row stride ldo).  splits > 1 divides every token's
 * keys over that many blocks which meet in `scratch` (b200_sink_attn_scratch_bytes) and are merged in index order. */
typedef struct b200_sink_attn_args {
    float* proj;
    int32_t ldp, q_off, k_off, v_off, g_off;
    const float* bias;
    const float* q_gain;
    const float* k_gain;
    const float* temp;
    const float* vmix;
    float* v_first;
    int32_t ldvf, vmix_mode;
    void* k_cache;
    void* v_cache;
    const uint64_t* kv_ptrs;
    const int32_t* pos;
    int32_t kv_ptr_stride, pos0;
    int32_t T, heads, kv_heads, dim, vdim, row_elems, cache_dtype;
    float eps, scale, sink;
    void* out;
    int32_t ldo, out_dtype;
    int32_t pdl, ldq16;
    void* q16;            /* optional: b200_sink_attn_append also leaves the finished queries here, in the cache's 16-bit type
                             ([T, heads * dim], row stride ldq16), for a kernel that reads its queries by TMA */
} b200_sink_attn_args;
int b200_sink_attn_append(const b200_sink_attn_args* args, void* stream);
int b200_sink_attn(const b200_sink_attn_args* args, int32_t splits, float* scratch, void* stream);
int64_t b200_sink_attn_scratch_bytes(int32_t T, int32_t heads, int32_t vdim, int32_t splits);
/* The same attention for a prompt-size chunk of ONE session on the tensor cores (16-bit caches and output, vdim <= 256;
 * k_cache / v_cache and pos0, not the pointer table): mma.sync m16n8k16 flash attention over the session's planes, scores and softmax fp32, the weights
 * enter P.V as two 16-bit terms.  Queries as b200_sink_attn_append left them. */
int b200_sink_attn_prefill(const b200_sink_attn_args* args, void* stream);

/* Gated delta rule behind short causal convolutions.  Rows r = s * seq_len + i: token i of sequence s (a decode step has
 * n_seq sequences of one token, a chunk of a prompt one sequence of seq_len tokens); position p = (pos ? pos[s] : pos0) + i.
 * proj[r] (fp32 row of the fused projection): the convolutions' inputs [q | k | v] (kv_heads*dim, kv_heads*dim, heads*vdim
 * channels) at c_off, one beta logit per head at b_off, one decay input per head at a_off.
 * A sequence's state (fp32, at state_ptrs ? state_ptrs[s * state_ptr_stride] : state, plus state_off elements):
 * [2][heads][vdim][dim] matrices (column-major) - a launch whose first token is at p0 reads copy p0 & 1 (zeros when p0 = 0) and writes copy
 * (p0 + seq_len) & 1 - followed by a ring [taps][channels] of convolution inputs, slot = position mod taps.
 * Step 1, b200_delta_prep (one warp or block per head and group of rows): y_c = silu(sum_b w[c][taps-1-b] x_c(p - b)), inputs before the sequence's
 * start are zero, inputs before the launch's first row come from the ring; q and k heads become unit vectors
 * x / sqrt(sum x^2 + unit_eps), q also times dim^-1/2; beta = sigmoid(.), decay = exp(-exp(A_log) softplus(. + dt_bias)).
 * work[r] = [q | k | v | beta | decay | k.q per key head] (fp32, row stride ldw >= channels + 2 heads + kv_heads).
 * Step 2, b200_delta_rule (sequential over a sequence's tokens, parallel over sequences, heads and columns):
 *   S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q      (head h uses q/k head h / (heads / kv_heads))
 * o: fp32 [rows, heads * vdim] (row stride ldo).  Also stores the last rows' convolution inputs in the ring. */
typedef struct b200_delta_args {
    const float* proj;
    int32_t ldp, c_off, b_off, a_off;
    const float* conv_w;      /* fp32 [channels, taps] */
    const float* A_log;
    const float* dt_bias;
    float* work;
    int32_t ldw;
    float* state;
    const uint64_t* state_ptrs;
    int32_t state_ptr_stride, reserved0;
    int64_t state_off;
    const int32_t* pos;
    int32_t pos0;
    int32_t n_seq, seq_len, heads, kv_heads, dim, vdim, taps;
    float unit_eps;
    float* o;
    int32_t ldo, pdl;
} b200_delta_args;
int b200_delta_prep(const b200_delta_args* args, void* stream);
int b200_delta_rule(const b200_delta_args* args, void* stream);

/* x[t, h, :] *= sigmoid(gate[t, h]) in place; x: 16-bit or fp32 [T, heads * vdim] (row stride ldx), gate: fp32 (row stride ldg). */
int b200_head_gate(void* x, int32_t ldx, int32_t dtype, const float* gate, int32_t ldg, int32_t T, int32_t heads, int32_t vdim,
                   int32_t pdl, void* stream);

/* Gated RMS norm per head: out[t, h, :] = o[t, h, :] / sqrt(mean(o^2) + eps) * gain[:] * silu(gate[t, h, :]).
 * o: fp32 [T, heads * vdim] (ldo); gate: fp32 rows (ldg) holding heads * vdim logits; gain: fp32 [vdim] shared by the
 * heads; out 16-bit or fp32 (ldout). */
int b200_gated_head_norm(const float* o, int32_t ldo, const float* gate, int32_t ldg, const float* gain, void* out,
                         int32_t ldout, int32_t out_dtype, int32_t T, int32_t heads, int32_t vdim, float eps, int32_t pdl,
                         void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_PETALS_H_ */
