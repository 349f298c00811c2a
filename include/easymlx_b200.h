/*
 * easymlx_b200 - C ABI of the B200 (sm_100a) ragged paged-attention path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as
 * void*), launches asynchronously on that stream and returns an emlx_status.  Nothing
 * here allocates or frees device memory unless its comment says so; the caller owns all
 * buffers.  After a non-zero return emlx_last_error() describes the failure (per host
 * thread).
 *
 * The comments cite the easymlx function each entry point replaces; paths are relative
 * to lib/python/easymlx/ in that project.
 */
#ifndef EASYMLX_B200_H
#define EASYMLX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

typedef enum emlx_status {
    EMLX_OK = 0,
    EMLX_ERR_INVALID = 1,     /* bad rank/shape/geometry  -> ValueError in the Python mirror        */
    EMLX_ERR_UNSUPPORTED = 2, /* geometry a kernel does not cover -> NotImplementedError            */
    EMLX_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed -> RuntimeError                   */
    EMLX_ERR_WORKSPACE = 4,   /* plan/workspace buffer missing or too small -> RuntimeError          */
    EMLX_ERR_DEVICE = 5       /* the device status word holds an error (see emlx_read_status)        */
} emlx_status;

/* Element types of queries / new rows / 16- and 32-bit pools. */
typedef enum emlx_dtype { EMLX_F16 = 0, EMLX_BF16 = 1, EMLX_F32 = 2 } emlx_dtype;

/* Storage format of the page pool.
 *   FLOAT   : key_cache/value_cache[NB, bs, Hkv, D] in `kv_dtype` (the reference layout,
 *             caching/paged/cache.py:779-791).
 *   AFFINE8 / AFFINE4 : min-max affine codes over groups of 64 along head_dim.
 *             key codes   uint8 [NB, bs, Hkv, D*bits/8]  (token-major, low nibble = even element)
 *             value codes uint8 [NB, Hkv, D, bs*bits/8]  (transposed inside a page: the tokens of one
 *                               head_dim element are contiguous; low nibble = even token)
 *             scale, bias fp16  [NB, Hkv, bs, D/64] for keys and for values.
 *             The reference has no such cache; its hook for a quantised cache is the k_scale/v_scale
 *             pair of operations/kernels/unified_attention.py:1391-1392.
 */
typedef enum emlx_kv_format { EMLX_KV_FLOAT = 0, EMLX_KV_AFFINE8 = 8, EMLX_KV_AFFINE4 = 4 } emlx_kv_format;

/* Bits of the device status word (int32, caller-allocated, zeroed by the caller). Kernels OR bits in. */
enum {
    EMLX_DEV_BAD_SLOT = 1,        /* slot id outside [0, num_slots)                                   */
    EMLX_DEV_BAD_PAGE = 2,        /* page id outside [0, num_blocks) inside a sequence's live range   */
    EMLX_DEV_OVERFLOW = 4,        /* a sequence would outgrow its page-table row                      */
    EMLX_DEV_TOKEN_MISMATCH = 8,  /* sum(query_lens) != total_tokens                                  */
    EMLX_DEV_WAIT_TIMEOUT = 16    /* an in-kernel barrier wait hit its iteration limit                */
};

/* The page pool, shared by the write and attention entry points. */
typedef struct emlx_pool {
    void* key_cache;      /* see emlx_kv_format                                      */
    void* value_cache;
    void* k_scale;        /* AFFINE only, else NULL                                  */
    void* k_bias;
    void* v_scale;
    void* v_bias;
    int64_t num_blocks;   /* NB                                                      */
    int32_t block_size;   /* bs, tokens per page                                     */
    int32_t num_kv_heads; /* Hkv                                                     */
    int32_t head_dim;     /* D                                                       */
    int32_t kv_format;    /* emlx_kv_format                                          */
    int32_t kv_dtype;     /* emlx_dtype of a FLOAT pool                              */
    int32_t reserved;
} emlx_pool;

/* One attention call: packed queries over already-gathered per-sequence rows.
 * Mirrors the arguments of paged_attention(), operations/kernels/unified_attention.py:1377-1393. */
typedef struct emlx_attn_args {
    const void* queries;            /* [T, Hq, D] q_dtype                             */
    void* out;                      /* [T, Hq, D] q_dtype, fully overwritten          */
    const int32_t* block_tables;    /* [S, MB], -1 = unassigned                       */
    const int32_t* kv_lens;         /* [S], lengths AFTER this step's write           */
    const int32_t* query_start_loc; /* [S+1]                                          */
    int32_t total_tokens;           /* T                                              */
    int32_t num_seqs;               /* S                                              */
    int32_t num_q_heads;            /* Hq, multiple of Hkv                            */
    int32_t max_blocks_per_seq;     /* MB                                             */
    int32_t q_dtype;                /* emlx_dtype                                     */
    int32_t sliding_window;         /* 0 = off                                        */
    float softmax_scale;
    int32_t max_query_len;          /* host hint: upper bound of query tokens per sequence, 0 = unknown */
    int32_t row_class_mask;         /* host hint: OR of 1 << emlx_attn_row_class(q_len) over the batch's query
                                     * lengths; kernels of the other row classes are not launched; 0 = unknown */
    int32_t plan_flags;             /* the plan_flags `plan` was built with (emlx_attn_plan / emlx_build_metadata):
                                     * they decide which row classes the plan holds, so the launch must use the same */
    void* plan;                     /* from emlx_attn_plan (not used by emlx_attn_generic)        */
    size_t plan_bytes;
    void* workspace;                /* split-KV partials and counters; zero it once after allocating, and again
                                     * after a call that reported EMLX_DEV_WAIT_TIMEOUT (counters may be left set) */
    size_t workspace_bytes;
    int32_t* status;                /* device status word, may be NULL                */
} emlx_attn_args;

const char* emlx_last_error(void);
int emlx_abi_version(void);

/* Blocking read of a device status word (synchronises `stream`). Returns EMLX_OK when it is 0,
 * EMLX_ERR_DEVICE otherwise with the bits spelled out in emlx_last_error(). */
int emlx_read_status(const int32_t* status, void* stream);

/* (2) Batch metadata on the GPU.  Replaces the host code of PageCacheView.concatenate_to_cache
 * (caching/paged/cache.py:1123-1169,1214-1261,1300-1305), build_query_start_loc
 * (caching/paged/cache.py:1448-1465) and the row gather of PageMetadata.with_cache_state
 * (caching/paged/cache.py:1201-1205,1301-1305).
 *   query_lens[S], slot_ids[S]             packed batch, in batch order (negative lengths count as 0)
 *   block_tables_all[num_slots, MB]        the cache's page table
 *   kv_lens_all[num_slots]                 in/out: advanced by query_lens when advance_kv_lens != 0
 *   query_start_loc[S+1]                   out: exclusive prefix sum of query_lens
 *   block_tables[S, MB], kv_lens[S]        out: rows of the scheduled slots, lengths after the step
 *   slot_mapping[T]                        out: page*bs + offset of every new row, -1 = skip
 * A slot id must not appear twice in one batch.  A sequence that would outgrow its page-table row sets
 * EMLX_DEV_OVERFLOW and is left alone: its stored length stays, its rows get slot_mapping -1 and kv_lens[i] = 0.
 * Ordering: all kernels of this library are launched with programmatic stream serialisation and wait for the
 * preceding launch of the stream before their first global load, so inputs produced by any earlier work of the
 * same stream (a projection, a copy, a previous step) are complete when they are read. */
int emlx_build_metadata(const int32_t* query_lens, const int32_t* slot_ids, int32_t num_seqs, int32_t total_tokens,
                        const int32_t* block_tables_all, int32_t num_slots, int32_t max_blocks_per_seq,
                        int32_t* kv_lens_all, int32_t block_size, int32_t advance_kv_lens,
                        int32_t* query_start_loc, int32_t* block_tables, int32_t* kv_lens, int64_t* slot_mapping,
                        int32_t* token_positions /* out, [T], position of every new row in its sequence; may be NULL */,
                        int64_t num_blocks, int32_t* status,
                        /* optional: also build the attention work list in the same launch (plan == NULL: skip) */
                        int32_t num_q_heads, int32_t num_kv_heads, int32_t sliding_window, int32_t max_query_len,
                        int32_t plan_flags, void* plan, size_t plan_bytes, void* stream);

/* (1) Paged KV write.  Replaces the scatter of PageCacheView.concatenate_to_cache
 * (caching/paged/cache.py:1186-1190,1278-1282) and, for AFFINE pools, the quantised-write hook
 * (caching/paged/cache.py:1171-1184).  keys/values are [T, Hkv, D] in `in_dtype`, contiguous. */
int emlx_kv_write(const void* keys, const void* values, int32_t in_dtype, int32_t total_tokens,
                  const int64_t* slot_mapping, const emlx_pool* pool, int32_t* status, void* stream);

/* Rotary embedding parameters: angle of pair i at position p is p * position_scale / freqs[i] with
 * inv_freq[i] = 1 / freqs[i]; pairs are (i, i + dims/2), or (2i, 2i+1) when `traditional`; the rotated slice is
 * multiplied by mscale.  Covers the reference's default / linear / llama3 / yarn variants, which all reduce to
 * mx.fast.rope(x, dims, traditional, base | freqs, scale, offset) (layers/rotary/_rotary.py:123-131,213-221,369-370). */
typedef struct emlx_rope {
    const float* inv_freq;        /* device, [dims / 2]                                     */
    int32_t dims;                 /* rotated leading dimensions of every head, even, <= D   */
    int32_t traditional;
    float position_scale;
    float mscale;
    int32_t head_dim_if_no_pool;  /* row width when emlx_kv_write_rope is called without a pool */
    int32_t reserved;
} emlx_rope;

/* (1)+(f1) Paged KV write with the rotary embedding fused in.  Replaces the RoPE calls inside
 * PageCacheView.concatenate_to_cache (caching/paged/cache.py:1161-1166,1225-1231) together with the scatter:
 * keys are rotated at token_positions[t] as they are read and then stored / quantised; queries are rotated into
 * queries_out in the same launch (queries_out == NULL: keys only; pool == NULL: queries only). */
int emlx_kv_write_rope(const void* queries, void* queries_out, int32_t num_q_heads, const void* keys,
                       const void* values, int32_t in_dtype, int32_t total_tokens, const int64_t* slot_mapping,
                       const int32_t* token_positions, const emlx_rope* rope, const emlx_pool* pool, int32_t* status,
                       void* stream);

/* (1)+(2) in ONE launch: batch metadata, the attention work list and the paged KV write of one step.  Replaces
 * PageCacheView.concatenate_to_cache as a whole (caching/paged/cache.py:1123-1306: the decode fast path :1155-1206 and
 * the ragged path :1208-1306).  Token j of sequence i goes to position kv_lens_all[slot_ids[i]] + j of its slot (page
 * block_tables_all[slot, pos / bs], offset pos % bs); the stored length grows by the sequence's query length (when
 * advance_kv_lens != 0); outputs as emlx_build_metadata: query_start_loc[S+1], block_tables[S, MB], kv_lens[S] (lengths
 * after the step) and, when plan != NULL, the attention work list (as emlx_attn_plan).
 *   query_lens[S]   device; NULL = every sequence has exactly one token (then total_tokens == num_seqs)
 *   keys/values     [T, Hkv, D] in in_dtype
 * With `rope` the keys are rotated at their positions before they are stored and, when queries_out != NULL, queries
 * [T, Hq, D] are rotated into queries_out (caching/paged/cache.py:1161-1166,1225-1231).
 * `ticket` is one int32 of device memory owned by the caller, zero before the first call; the kernel leaves it zero.
 * A slot id must not appear twice.  A sequence that would outgrow its page-table row sets EMLX_DEV_OVERFLOW, keeps its
 * stored length, writes nothing and gets kv_lens[i] = 0 (attention then returns zero rows for it).  Up to 2048
 * sequences; larger batches return EMLX_ERR_UNSUPPORTED and go through emlx_build_metadata + emlx_kv_write. */
int emlx_kv_write_step(const void* queries, void* queries_out, const void* keys, const void* values, int32_t in_dtype,
                       const int32_t* query_lens, const int32_t* slot_ids, int32_t num_seqs, int32_t total_tokens,
                       const int32_t* block_tables_all, int32_t num_slots, int32_t max_blocks_per_seq,
                       int32_t* kv_lens_all, int32_t advance_kv_lens, const emlx_pool* pool, const emlx_rope* rope,
                       int32_t* query_start_loc, int32_t* block_tables, int32_t* kv_lens, int32_t num_q_heads,
                       int32_t sliding_window, int32_t max_query_len, int32_t plan_flags, void* plan, size_t plan_bytes,
                       int32_t* ticket, int32_t* status, void* stream);
/* The same for a batch in which every scheduled sequence appends exactly one token (query_lens == NULL above): the
 * decode fast path of concatenate_to_cache (caching/paged/cache.py:1155-1206). */
int emlx_kv_write_decode(const void* queries, void* queries_out, const void* keys, const void* values, int32_t in_dtype,
                         const int32_t* slot_ids, int32_t num_seqs, const int32_t* block_tables_all, int32_t num_slots,
                         int32_t max_blocks_per_seq, int32_t* kv_lens_all, int32_t advance_kv_lens, const emlx_pool* pool,
                         const emlx_rope* rope, int32_t* query_start_loc, int32_t* block_tables, int32_t* kv_lens,
                         int32_t num_q_heads, int32_t sliding_window, int32_t plan_flags, void* plan, size_t plan_bytes,
                         int32_t* ticket, int32_t* status, void* stream);

/* Work list for the tiled attention kernels, built on the GPU from query_start_loc / kv_lens
 * (replaces the host-side classification of _is_single_token_decode,
 * operations/kernels/unified_attention.py:175-184, which forces a device->host sync). */
size_t emlx_attn_plan_bytes(int32_t num_seqs, int32_t total_tokens, int32_t num_q_heads, int32_t num_kv_heads);
size_t emlx_attn_workspace_bytes(int32_t num_seqs, int32_t total_tokens, int32_t num_q_heads, int32_t num_kv_heads,
                                 int32_t head_dim);
int emlx_attn_plan(const int32_t* query_start_loc, const int32_t* kv_lens, int32_t num_seqs, int32_t total_tokens,
                   int32_t num_q_heads, int32_t num_kv_heads, int32_t block_size, int32_t sliding_window,
                   int32_t max_query_len /* host hint, 0 = unknown */, int32_t plan_flags /* emlx_attn_plan_flags() */,
                   void* plan, size_t plan_bytes, void* stream);
/* Flags a plan should be built with for this pool and head geometry: bit 0 = cut sequences with more than 32
 * query rows into 128-row units for the tcgen05 prefill kernel (fp16/bf16 pools, 128 % (Hq/Hkv) == 0).
 * Bit 1 = the 8-row kernel runs two CTAs per SM and its slices are cut for twice as many CTAs (4-bit pools,
 * where unpacking the codes, not HBM, limits what one CTA's warps get through).
 * Bits 8-15 (a tuning knob, normally 0): in a batch that holds both short rows and 128-row units the short-row
 * kernel and the 128-row kernel run side by side, the former on a share of the SMs that the work list chooses from the
 * two amounts of work; a non-zero value here fixes that share (in CTAs) instead. */
int emlx_attn_plan_flags(int32_t kv_format, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim);
/* Row class (0..3: which kernel variant serves it) of a sequence with `query_len` tokens in this step, for
 * emlx_attn_args.row_class_mask; -1 for query_len <= 0 (such sequences produce no rows). */
int emlx_attn_row_class(int32_t kv_format, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, int32_t query_len);

/* (5) Unified ragged attention: decode rows and prefill chunks of one packed batch in one call.
 * Replaces paged_attention() (operations/kernels/unified_attention.py:1377-1512) and the Metal
 * kernels it launches (unified_attention.py:290-464, 467-608). */
int emlx_attn_unified(const emlx_attn_args* args, const emlx_pool* pool, void* stream);
/* (3) Split-KV flash-decode over the plan's short-row units only (row classes 0-2: up to 32 query rows per unit).
 * EMLX_ERR_UNSUPPORTED when the plan can hold no such unit (a plan built with 128-row units and a GQA group above
 * 16 puts even single-token rows into class 3): `out` is then left untouched. */
int emlx_attn_decode(const emlx_attn_args* args, const emlx_pool* pool, void* stream);
/* (4) Prefill-chunk attention over the plan's long-row units only (row class 3, 128-row units; needs a plan built
 * with emlx_attn_plan_flags() bit 0).  EMLX_ERR_UNSUPPORTED when the plan holds no such class. */
int emlx_attn_prefill(const emlx_attn_args* args, const emlx_pool* pool, void* stream);
/* Reference-semantics kernel for any geometry the tiled kernels do not cover (head_dim <= 256,
 * any page size, fp16/bf16/fp32); same arithmetic as _paged_attention_reference
 * (operations/kernels/unified_attention.py:187-281).  Needs neither plan nor workspace. */
int emlx_attn_generic(const emlx_attn_args* args, const emlx_pool* pool, void* stream);

/* Prefill chunks over an affine (8/4-bit) pool on the tcgen05 kernel.  With plan_flags bit 0 set for an affine pool
 * (128 % (Hq/Hkv) == 0, head_dim 64/128), emlx_attn_unified first expands the pages of the sequences that own 128-row
 * units (more than 16 rows) to 16-bit rows in scratch memory and runs the 128-row kernel over those; the other rows
 * read the codes as before.  The scratch sits directly behind the workspace: pass a workspace of
 * emlx_attn_workspace_bytes(...) + emlx_attn_dequant_bytes(pool, num_seqs, max_blocks_per_seq, n, total_tokens,
 * num_q_heads, q_dtype) bytes (zeroed once, like the workspace), n = an upper bound on the sequences with more than
 * 16 rows in the batch.  The expanded rows are fp16; for bf16 queries the scratch also holds fp16 copies of those
 * sequences' queries and output rows (the tensor core multiplies operands of one type), converted on the way in and out.  A batch that holds
 * more such sequences sets EMLX_DEV_OVERFLOW in *status (their rows come out as zeros).  The expanded pages are not
 * cleaned up: a caller that reuses the buffer for a call of another geometry (whose workspace part ends elsewhere)
 * zeroes the first emlx_attn_workspace_bytes() bytes again before that call.  The reference serves a quantised cache through the
 * same route for every row kind (operations/kernels/unified_attention.py:1633-1656). */
size_t emlx_attn_dequant_bytes(const emlx_pool* pool, int32_t num_seqs, int32_t max_blocks_per_seq, int32_t num_long_seqs,
                               int32_t total_tokens, int32_t num_q_heads, int32_t q_dtype);

/* Decode attention without caller-provided scratch.  No counterpart in the reference.
 * For embedders that cannot allocate device memory around this call: a serving process whose allocator has
 * already reserved all of HBM (a later cudaMalloc for the work list or the split-KV workspace could fail or
 * fragment the pool), or a step loop that must not take the device-wide synchronisation cudaMalloc/cudaFree
 * imply.  Same result as emlx_attn_plan + emlx_attn_decode; args->plan/workspace are ignored and the entry
 * point builds the work list itself.  Scratch is a 12 MiB array built into the library (held by every GPU the
 * library runs on until the process exits); a batch whose plan + workspace exceed it is rejected with
 * EMLX_ERR_WORKSPACE (in practice: up to a few thousand sequences / tokens).  The first call on a device looks
 * up the array's address; make that first call outside any stream capture.  All calls share the array: two
 * calls that overlap on the GPU (different streams) race, so serialise them.  Calls no allocating routine. */
int emlx_attn_decode_static(const emlx_attn_args* args, const emlx_pool* pool, void* stream);

/* ---- KV heads sharded over GPUs: attention whose epilogue gathers the output over peer-mapped memory ----------------
 * No counterpart in the reference (eSurge runs one device; its multi-device code is a replicated control plane,
 * inference/esurge/distributed/).  One process per GPU; rank r holds the pages of KV heads [r*Hkv/N, (r+1)*Hkv/N) of
 * every sequence and computes the query heads that belong to them.  Instead of an all-gather of the [T, Hq/N, D]
 * slices afterwards, the kernels store every finished row straight into the full [T, Hq, D] output buffer of every
 * rank (plain stores through peer-mapped pointers; no TMA, no multicast on peer memory) and exchange two flags per
 * pair of ranks: "my output buffer may be overwritten" at the start of a call and "my rows have arrived" at its end.
 * Both waits are bounded by `poll_limit` polls; on expiry the kernel ORs EMLX_DEV_WAIT_TIMEOUT into *status and
 * finishes.  All ranks must make the same sequence of gathering calls (same batch, one call per step); whatever
 * reads the output must be queued on the calling stream before the rank's next gathering call. */
#define EMLX_MAX_PEERS 8
#define EMLX_PEER_FLAG_BYTES 512   /* one rank's flag block; allocate it in peer-shared memory and zero it once */
#define EMLX_PEER_HANDLE_BYTES 64
/* Device memory that other processes on the same node can map: create (cudaMalloc + zero + IPC handle), open a
 * handle received from another rank, close a mapping, free an own buffer.  Exchange the handles over any host
 * channel (torch.distributed all_gather of 64 bytes). */
int emlx_peer_buffer_create(size_t bytes, void** ptr, void* handle);
int emlx_peer_buffer_open(const void* handle, void** ptr);
int emlx_peer_buffer_close(void* ptr);
int emlx_peer_buffer_free(void* ptr);
/* Writes the table of the ranks' output buffers and flag blocks (as mapped into this process; entry `rank` is the
 * local one) into this rank's flag block.  Call once after the handles are exchanged, before the first gathering
 * call, with the flag block zeroed. */
int emlx_gather_init(void* flag_block, void* const* out_ptrs, void* const* flag_ptrs, int32_t num_ranks, int32_t rank,
                     int32_t poll_limit, void* stream);
/* emlx_attn_decode over this rank's heads (args->num_q_heads = Hq/N, pool = this rank's KV heads; the work list must
 * be built without 128-row units, plan_flags bit 0 clear), writing heads [head_offset, head_offset + Hq/N) of
 * args->out = this rank's full [T, total_q_heads, D] buffer and of every other rank's. */
int emlx_attn_decode_gather(const emlx_attn_args* args, const emlx_pool* pool, void* flag_block, int32_t total_q_heads,
                            int32_t head_offset, void* stream);

/* Failure-detection self-test: launches one warp that waits, with the kernels' bounded-wait routine and a limit of
 * `poll_limit` polls, on a barrier that is never completed; the wait gives up, the kernel ORs EMLX_DEV_WAIT_TIMEOUT
 * into *status and returns normally (nothing faults, the context stays usable). */
int emlx_selftest_wait_timeout(int32_t* status, uint32_t poll_limit, void* stream);

/* Host-only self-test of the per-device set-up bookkeeping (kernel attributes such as the dynamic shared-memory limit
 * and the SM count are kept once per device ordinal, so one process can drive several GPUs).  Makes no CUDA call;
 * returns the number of failed checks (0 = pass). */
int emlx_selftest_device_once(void);

/* ---- batch and page-table maintenance on the device (no host synchronisation; bound by HBM or launch latency) ---- */

/* out[s] = rows[query_start_loc[s+1] - 1] for s in [0, S): the last token's row of every sequence of a packed
 * [T, row_bytes] array (hidden states).  Replaces _extract_last_tokens, modules/_base/causal_lm_module.py:176-207
 * (take at qsl[1:] - 1; an index of -1 wraps to the last row as mx.take does).  An index outside [0, T) sets
 * EMLX_DEV_TOKEN_MISMATCH in *status (may be NULL) and leaves that output row untouched. */
int emlx_gather_last_tokens(const void* rows, int32_t total_tokens, int64_t row_bytes, const int32_t* query_start_loc,
                            int32_t num_seqs, void* out, int32_t* status, void* stream);

/* out[s, i] = i < len(s) ? flat_ids[query_start_loc[s] + i] : 0, out is int32 [S, max_query_len].  Replaces the
 * compiled batch padder of inference/esurge/runners/model_runner.py:1250-1269. */
int emlx_pad_token_ids(const int32_t* flat_ids, int32_t total_tokens, const int32_t* query_start_loc, int32_t num_seqs,
                       int32_t max_query_len, int32_t* out, void* stream);

/* Copy-on-write page copies: for every (src, dst) row of block_mapping [num_pairs, 2] (device, int32) copy page src to
 * page dst in every array of the pool (codes, and scales / biases of an affine pool).  Replaces
 * PageCacheView.copy_blocks, caching/paged/cache.py:944-972, whose kernel reads every source from the pool as it
 * was before the call.  With `staging` (device, 16-byte aligned, num_pairs * emlx_page_staging_bytes(pool) bytes)
 * the copy keeps exactly that meaning for any mapping (two launches through the staging area); with staging == NULL
 * pages are copied in place in one launch, which is only equivalent when no page is both a source and a
 * destination and no destination repeats.  A page id outside [0, NB) skips its pair and sets EMLX_DEV_BAD_PAGE. */
int64_t emlx_page_staging_bytes(const emlx_pool* pool);
int emlx_copy_blocks(const emlx_pool* pool, const int32_t* block_mapping, int32_t num_pairs, void* staging,
                     int64_t staging_bytes, int32_t* status, void* stream);

/* Contiguous K/V of the listed sequences: k_out / v_out [total_tokens, Hkv, D] in out_dtype, token t of sequence s read
 * from page block_table[s, (t - cu_seq_lens[s]) / bs].  Float pools are cast, affine pools dequantised
 * (scale * code + bias in fp32).  Replaces PageCacheView.gather_kv_cache, caching/paged/cache.py:974-1027 (whose kernel
 * reads the packed side caches this build does not keep) and, with one row per page, the whole-pool dequantisation of
 * dequantize_kv_cache, cache.py:1050-1086.  A page id outside [0, NB) leaves zero rows and sets EMLX_DEV_BAD_PAGE. */
int emlx_gather_kv_cache(const emlx_pool* pool, const int32_t* block_table, int32_t num_seqs, int32_t max_blocks_per_seq,
                         const int32_t* cu_seq_lens, int32_t total_tokens, int32_t out_dtype, void* k_out, void* v_out,
                         int32_t* status, void* stream);

/* Zero pages page_ids[0..count) (device, int32) in every array of the pool; ids outside [0, NB) are skipped, as
 * _zero_pages does (inference/esurge/runners/model_runner.py:1058-1094). */
int emlx_zero_pages(const emlx_pool* pool, const int32_t* page_ids, int32_t count, void* stream);

/* block_tables[row, :] = -1; block_tables[row, :count] = page_ids (device, count clipped to MB);
 * kv_lens[row] = max(cached_tokens, 0).  Replaces _assign_row_mapping, model_runner.py:1096-1131; a row outside
 * the table is EMLX_ERR_INVALID (the reference raises RuntimeError). */
int emlx_rows_assign(int32_t* block_tables, int32_t* kv_lens, int32_t num_slots, int32_t max_blocks_per_seq, int32_t row,
                     const int32_t* page_ids, int32_t count, int32_t cached_tokens, void* stream);

/* Apply `count` row operations in order.  mode 0: ops is [count, 2] (from, to) and each pair moves row `from` onto
 * row `to`, then clears `from` (table row = -1, length = 0): compact_rows, model_runner.py:1215-1241.  mode 1: each
 * pair swaps the two rows: _move_cache_row, model_runner.py:1192-1213.  mode 2: ops is [count] rows to clear:
 * _clear_row_mapping, model_runner.py:1010-1025.  Rows outside the table are skipped and set EMLX_DEV_BAD_SLOT. */
int emlx_rows_update(int32_t* block_tables, int32_t* kv_lens, int32_t num_slots, int32_t max_blocks_per_seq,
                     const int32_t* ops, int32_t count, int32_t mode, int32_t* status, void* stream);

/* Number of kernels this library has launched from the calling process.  A benchmark that reports how many of
 * the library's kernels ran in its timed region reads it before and after. */
int64_t emlx_launch_count(void);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* EASYMLX_B200_H */
