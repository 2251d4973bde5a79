/*
 * q4_gpu.h -- C ABI of libq4gpu: the KV-cache + attention hot path of the q4 inference engine,
 * implemented as hand-written CUDA for NVIDIA B200 (sm_100a).
 *
 * Two groups of entry points:
 *
 *  1. `q4_hip_*` -- the reference engine's own device ABI for this path, exported under the
 *     same names, parameter lists and conventions (each cites the declaration it replaces in
 *     the reference's src/q4.h and the implementation in src/q4_rocm.cu), so the C host
 *     (src/q4_fwd.c, src/q4_mtp.c, src/q4_test.c) links against libq4gpu unchanged.  These
 *     operate on caller-owned caches in the reference layout
 *     [token][kv_head][hd/32 x {fp16 scale, 32 x int8}] (q8_0), or fp16 / fp32 rows.
 *
 *  2. `q4_gpu_*` -- additive entry points: a library-owned KV store with a B200-native record
 *     layout, fused K+V append, batched multi-session decode, bf16 queries, per-kv-head
 *     selection lists, partial (m, l, acc) output + merge for sequence-sharded decode,
 *     tensor-core prefill, and bulk prefix save/restore.
 *
 * Conventions (inherited from the reference, src/q4_rocm.cu:20-28,52-57,202-214):
 *  - every operation returns bool: true = enqueued, false = rejected (bad argument, library not
 *    initialised, launch failure); NULL / zero-size arguments return false and never crash;
 *  - all work is asynchronous on ONE internal compute stream and ordered by it; only
 *    q4_hip_h2d / q4_hip_d2h (outside capture), q4_hip_stream_sync and q4_hip_sync block;
 *  - state is process-global and bound to one device (one process per GPU); the caller is
 *    single-threaded with respect to launches;
 *  - device pointers passed in are owned by the caller, scratch by the library;
 *  - `kind` (the reference's `kv_f16` argument): 0 = fp32 rows, 1 = fp16 rows, 2 = q8_0;
 *  - there is no CPU fallback: without a CUDA device q4_hip_init() returns false and every
 *    other call fails.
 */
#ifndef Q4_GPU_H
#define Q4_GPU_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ======================================================================================= */
/* 1. Reference ABI (drop-in)                                                               */
/* ======================================================================================= */

/* src/q4.h:708-710, src/q4_rocm.cu:88-120.  Device = $Q4_GPU_DEVICE, else $LOCAL_RANK, else 0. */
bool q4_hip_init(void);
void q4_hip_shutdown(void);
bool q4_hip_ok(void);

/* src/q4.h:877-880, src/q4_rocm.cu:300-322.  h2d/d2h are enqueued on the compute stream and,
 * outside graph capture, waited for. */
void *q4_hip_malloc(size_t n);
void q4_hip_free(void *p);
bool q4_hip_h2d(void *d, const void *h, size_t n);
bool q4_hip_d2h(void *h, const void *d, size_t n);
/* src/q4.h:787-789, src/q4_rocm.cu:8417-8432 */
bool q4_hip_d2h_async(void *h, const void *d, uint64_t n);
bool q4_hip_h2d_async(void *d, const void *h, uint64_t n);
bool q4_hip_stream_sync(void);
/* Upload on the separate copy stream and the blocking wait for it (src/q4.h:832,887,
 * src/q4_rocm.cu:247-250,3270-3275): lets the next step's inputs travel while this step computes. */
bool q4_hip_copy_h2d(void *dst, const void *src, size_t n);
void q4_hip_copy_wait(void);
/* src/q4.h:851,781, src/q4_rocm.cu:5656-5670 (n counts floats; copy is device-to-device) */
bool q4_hip_copy(float *d, const float *s, uint64_t n);
bool q4_hip_fill(float *d, float v, uint64_t n);
/* src/q4.h:948-949, src/q4_rocm.cu:292-298 */
void q4_hip_sync(void);
void q4_hip_clear(void);

/* Decode position word read by graph-captured kernels.  src/q4.h:686-688, src/q4_rocm.cu:6218-6227 */
void q4_hip_pos_push(int32_t pos);
int q4_hip_capturing(void);
int q4_hip_pos_dev_ok(void);

/* Stream capture of the compute stream.  src/q4.h:782-786, src/q4_rocm.cu:8162-8246 */
int q4_hip_graph_begin(void);
void *q4_hip_graph_end(void);
uint32_t q4_hip_graph_nodes(void *exec);
bool q4_hip_graph_launch(void *exec);
void q4_hip_graph_free(void *exec);

/* fp32 -> q8_0 blocks / fp16, n floats (n % 32 == 0 for q8).  src/q4.h:928-929,
 * src/q4_rocm.cu:7208-7247.  q8_0 codes and scales are bit-exact with the IEEE evaluation of the
 * reference quantiser. */
bool q4_hip_f32_to_f16(void *dst_f16, const float *src, uint64_t n);
bool q4_hip_f32_to_q8(void *dst_q8, const float *src, uint64_t n);
/* fp32 -> fp16 at row `*pos` of dst_base (row stride in elements).  src/q4.h:696-697,
 * src/q4_rocm.cu:7943-7958 */
bool q4_hip_f32_to_f16_d(void *dst_base, uint32_t stride_elems, const float *src, uint64_t n);
/* Append K and V (n floats each) at the token slot held in the device position word:
 * destination = cache + pos * bpt.  src/q4.h:694-695, src/q4_rocm.cu:7962-8012 */
bool q4_hip_kv_append_d(void *kcache, void *vcache, const float *k, const float *v, uint32_t n,
                        uint32_t bpt, int kind);

/* Per-head RMSNorm (+ weight), interleaved-pair RoPE on the first n_rot dims; q_prep also splits
 * the packed [q | gate] projection.  `_n` = n_tok rows at pos0 + t; `_d` = position from the
 * device word.  src/q4.h:689-693,895-905, src/q4_rocm.cu:6229-6343 */
bool q4_hip_qsa_q_prep(const float *d_qg, const float *d_wn, float *d_q, float *d_g,
                       uint32_t n_head, uint32_t hd, uint32_t n_rot, int32_t pos, float base,
                       float eps);
bool q4_hip_qsa_q_prep_n(const float *d_qg, const float *d_wn, float *d_q, float *d_g,
                         uint32_t n_head, uint32_t hd, uint32_t n_rot, int32_t pos0, float base,
                         float eps, uint32_t n_tok);
bool q4_hip_qsa_q_prep_d(const float *qg, const float *wn, float *q, float *g, uint32_t n_head,
                         uint32_t hd, uint32_t n_rot, float base, float eps);
bool q4_hip_qsa_k_prep(float *d_k, const float *d_wn, uint32_t n_kvh, uint32_t hd, uint32_t n_rot,
                       int32_t pos, float base, float eps);
bool q4_hip_qsa_k_prep_n(float *d_k, const float *d_wn, uint32_t n_kvh, uint32_t hd,
                         uint32_t n_rot, int32_t pos0, float base, float eps, uint32_t n_tok);
bool q4_hip_qsa_k_prep_d(float *k, const float *wn, uint32_t n_kvh, uint32_t hd, uint32_t n_rot,
                         float base, float eps);

/* GQA attention over the cache; out = softmax(q.k * scale) v * sigmoid(gate).
 *  decode    : one token over [0, n_kv)                      src/q4.h:621-624, q4_rocm.cu:8014-8022
 *  decode_n  : token t over [0, min(kv_base+t+1, max_kv))    src/q4.h:906-909, q4_rocm.cu:7249-7305
 *  decode_idx: token t over idx[t*width .. +width), -1 = skip  src/q4.h:911-915, q4_rocm.cu:7306-7364
 * q, gate, out: [n_tok][n_head][hd] fp32 on the device.  hd in {32,64,128,256}, n_head/n_kvh <= 16. */
bool q4_hip_qsa_decode(const float *d_q, const void *d_kcache, const void *d_vcache,
                       const float *d_gate, float *d_out, uint32_t n_head, uint32_t n_kvh,
                       uint32_t hd, uint32_t n_kv, uint32_t max_kv, float scale, int kv_f16);
bool q4_hip_qsa_decode_n(const float *d_q, const void *d_kcache, const void *d_vcache,
                         const float *d_gate, float *d_out, uint32_t n_head, uint32_t n_kvh,
                         uint32_t hd, uint32_t n_tok, uint32_t kv_base, uint32_t max_kv,
                         float scale, int kv_f16);
bool q4_hip_qsa_decode_idx(const float *d_q, const void *d_kcache, const void *d_vcache,
                           const float *d_gate, float *d_out, const int32_t *idx, uint32_t width,
                           uint32_t n_head, uint32_t n_kvh, uint32_t hd, uint32_t n_tok,
                           uint32_t max_kv, float scale, int kv_f16);
/* Pre-allocates the attention scratch (split-KV partials) so nothing allocates inside a capture.
 * src/q4.h:704, src/q4_rocm.cu:7698-7707 */
bool q4_hip_qsa_topk_alloc(void);

/* ---- QSA indexer (src/q4.h:698-706, 916-927; src/q4_rocm.cu:7366-7940): the producer of the `sel`
 * lists.  raw_f16: the indexer's fp16 key store [token][128]; pool: fp32 [block][128], block b =
 * mean of `ratio` keys, RMSNorm (wn, eps), RoPE at position b*ratio; score[t][b] = sum over the
 * n_head <= 4 indexer heads of relu(q[t][h] . pool[b]) for b < (pos0 + t + 1) / ratio, else -1e30;
 * topk: the min(n_vis, k_blk <= 512) best blocks by (score descending, index ascending) as positions
 * (blocks above the threshold in index order, then ties in index order), then the newest partial
 * block up to the token's position, then -1, `width` entries per token.  The _d forms take the
 * position from the device position word (graph-captured decode).  hd must be 128. */
bool q4_hip_qsa_pool(const void *raw_f16, float *pool, const float *wn, uint32_t hd, uint32_t ratio,
                     uint32_t b0, uint32_t b1, uint32_t n_rot, float rope_base, float eps);
bool q4_hip_qsa_pool_d(const void *raw, float *pool, const float *wn, uint32_t hd, uint32_t ratio,
                       uint32_t n_rot, float rope_base, float eps);
bool q4_hip_qsa_score(const float *q, const float *pool, float *score, uint32_t n_tok, uint32_t n_blocks,
                      uint32_t stride, uint32_t n_head, uint32_t hd, uint32_t pos0, uint32_t ratio);
bool q4_hip_qsa_score_d(const float *q, const float *pool, float *score, uint32_t stride, uint32_t n_head,
                        uint32_t hd, uint32_t ratio);
bool q4_hip_qsa_topk(const float *score, int32_t *sel, uint32_t n_tok, uint32_t n_blocks, uint32_t stride,
                     uint32_t k_blk, uint32_t ratio, uint32_t pos0, uint32_t width);
bool q4_hip_qsa_topk_d(const float *score, int32_t *sel, uint32_t stride, uint32_t k_blk, uint32_t ratio,
                       uint32_t width);

/* Batched indexer for concurrent sessions (additive): row t of q [n_sess][n_head][hd], score
 * [n_sess][stride] and sel [n_sess][width] belongs to session t, which has its own pool (pools[t]: a
 * device array of device pointers) and its own position (pos[t]: a device array, e.g. the one the
 * batch decode reads).  Two launches for all sessions; the same arithmetic and the same lists as one
 * q4_hip_qsa_score_d + q4_hip_qsa_topk_d pair per session (src/q4_fwd.c:894-920).  Every session must
 * have at most `stride` visible blocks.  The lists feed q4_gpu_batch_decode / _append_decode with
 * idx_kvh_stride 0 and idx_sess_stride width. */
bool q4_gpu_qsa_select_batch(const float *const *pools, const int32_t *pos, const float *q, float *score,
                             int32_t *sel, uint32_t n_sess, uint32_t stride, uint32_t n_head, uint32_t hd,
                             uint32_t k_blk, uint32_t ratio, uint32_t width);

/* ======================================================================================= */
/* 2. B200-native additions                                                                 */
/* ======================================================================================= */

/* Sticky status word of the last failed call / device-side check (0 = none); reading clears it.
 * Bits: 1 bad argument, 2 CUDA error, 4 out-of-range position seen by a kernel (the position was
 * skipped, nothing was accessed out of bounds), 8 scratch too small, 16 not initialised. */
uint32_t q4_gpu_last_error(void);
/* Internal compute stream as a cudaStream_t, and adoption of a caller's stream (NULL restores the
 * internal one).  No counterpart in the reference (its stream is private, src/q4_rocm.cu:52-54). */
void *q4_gpu_stream(void);
void *q4_gpu_copy_stream(void);   /* the copy stream as a cudaStream_t, for event ordering without a host wait */
/* Download on a third stream (no counterpart in the reference, which reads results back on its compute
 * stream): device-to-host copies overlap the next step's kernels and uploads.  Order it with events. */
bool q4_gpu_copy_d2h(void *dst, const void *src, size_t n);
void *q4_gpu_download_stream(void);
bool q4_gpu_set_stream(void *cuda_stream);
int q4_gpu_device(void);
/* A pipelined step loop over one set of step buffers (no counterpart in the reference, whose decode step
 * uploads, computes and reads back on one stream).  A host that decodes step after step from host buffers
 * keeps two or three sets of device input / output buffers, each with a captured graph that reads and writes
 * them; a pipe holds the events that order one set's upload (copy stream), graph (compute stream) and
 * download (download stream), so step i + 1 travels in while step i computes and step i - 1 travels out:
 *     q4_gpu_pipe_upload(next, ...); q4_gpu_pipe_run(this, graph, ...);   per step, nothing else.
 * upload: pinned host memory -> the set's device input buffer, after the set's previous graph launch.
 * run: the graph, after the set's upload and its previous download; then src_d -> dst_h (n bytes; n = 0: no
 * download).  Both return at once.  sync: blocks until the set's last download has landed. */
typedef struct q4_gpu_pipe q4_gpu_pipe;
q4_gpu_pipe *q4_gpu_pipe_create(void);
void q4_gpu_pipe_destroy(q4_gpu_pipe *p);
bool q4_gpu_pipe_upload(q4_gpu_pipe *p, void *dst_d, const void *src_h, size_t n);
bool q4_gpu_pipe_run(q4_gpu_pipe *p, void *graph_exec, void *dst_h, const void *src_d, size_t n);
bool q4_gpu_pipe_sync(q4_gpu_pipe *p);
/* Device address of the position word written by q4_hip_pos_push. */
const int32_t *q4_gpu_pos_word(void);

/* ---- KV store: allocator + layout (replaces q4_sess KV fields, kv_at, kv_token_bytes,
 * kv_write: src/q4_fwd.c:26-57,637-665,1944-1950; sizing q4_qsa_kv_bytes src/q4_place.c:92-105).
 * One store per session.  q8_0 layout: one record per (layer, kv head, position) holding the K codes,
 * the V codes, the K block scales and the V block scales (128 + 128 + 8 + 8 = 272 bytes at hd 128),
 * so a gathered position is one contiguous, 16-byte aligned read.  fp16 / fp32 kinds: K and V planes
 * of [layer][kv head][max_kv][hd] rows. */
typedef struct q4_gpu_kv q4_gpu_kv;
/* Device bytes q4_gpu_kv_create allocates for the K and V planes of such a store (what a placement
 * planner must reserve): equal to q4_qsa_kv_bytes at hd 128 / 256; q8_0 records at hd 32 / 64 are
 * padded to 16 bytes (80 instead of 68, 144 instead of 136 per kv head and position). */
uint64_t q4_gpu_kv_bytes(uint32_t n_layers, uint32_t n_kvh, uint32_t hd, uint32_t max_kv, int kind);
q4_gpu_kv *q4_gpu_kv_create(uint32_t n_layers, uint32_t n_kvh, uint32_t hd, uint32_t max_kv,
                            int kind);
void q4_gpu_kv_destroy(q4_gpu_kv *kv);
/* Fused K+V append of n_tok rows ([n_tok][n_kvh*hd] fp32, device) at token slots pos0.. of one
 * layer: quantise (q8_0) / convert / copy and scatter, one launch (replaces the two
 * q4_hip_f32_to_q8 launches of src/q4_fwd.c:823-824,1738-1741). */
bool q4_gpu_kv_append(q4_gpu_kv *kv, uint32_t layer, const float *k, const float *v, uint32_t pos0,
                      uint32_t n_tok);
/* Same for one token at the slot held in the device position word (replaces q4_hip_kv_append_d,
 * src/q4_fwd.c:891). */
bool q4_gpu_kv_append_d(q4_gpu_kv *kv, uint32_t layer, const float *k, const float *v);
/* K prep fused into the append: RMSNorm (optional weight) + interleaved-pair RoPE of the raw K rows,
 * then quantise / convert K and V and scatter them, one launch.  Replaces q4_hip_qsa_k_prep_{n,d}
 * followed by the append (src/q4_fwd.c:884,891 decode; :1734,1738-1741 prefill); the cache bytes are
 * those of that two-launch sequence.  k_raw, v: [n_tok][n_kvh*hd] fp32; k_raw is not modified. */
bool q4_gpu_kv_prep_append(q4_gpu_kv *kv, uint32_t layer, const float *k_raw, const float *v,
                           const float *k_norm_w, uint32_t n_rot, float rope_base, float eps,
                           uint32_t pos0, uint32_t n_tok);
bool q4_gpu_kv_prep_append_d(q4_gpu_kv *kv, uint32_t layer, const float *k_raw, const float *v,
                             const float *k_norm_w, uint32_t n_rot, float rope_base, float eps);
/* Rows [tok0, tok0+n_tok) of one layer's K (which = 0) or V (1) cache to / from the reference
 * layout (n_tok * kv_token_bytes device bytes) -- what q4_sess_save writes per layer,
 * src/q4_fwd.c:2353-2360. */
bool q4_gpu_kv_export(const q4_gpu_kv *kv, uint32_t layer, int which, uint32_t tok0, uint32_t n_tok,
                      void *dst);
bool q4_gpu_kv_import(q4_gpu_kv *kv, uint32_t layer, int which, uint32_t tok0, uint32_t n_tok,
                      const void *src);
/* Prefix snapshot (the KV part of q4_sess_save / q4_sess_restore, src/q4_fwd.c:2314-2477) as bulk
 * strided copies of rows [0, n_kv) of every plane.  buf is device memory (host = 0) or pinned /
 * pageable host memory (host = 1).  snapshot_bytes = n_kv * n_layers * n_kvh * bytes per (kv head,
 * position): 2*hd + hd/8 rounded up to 16 for q8_0 (at hd 128 / 256 that equals the reference's
 * n_kv * n_layers * 2 * kv_token_bytes; hd 32 / 64 records carry 12 / 8 bytes of padding), else the K and
 * V rows of hd fp16 / fp32 values. */
uint64_t q4_gpu_kv_snapshot_bytes(const q4_gpu_kv *kv, uint32_t n_kv);
bool q4_gpu_kv_save(const q4_gpu_kv *kv, uint32_t n_kv, void *buf, int host);
bool q4_gpu_kv_restore(q4_gpu_kv *kv, uint32_t n_kv, const void *buf, int host);

/* The KV section of the reference's session file, streamed to / from a file descriptor at its current
 * position (which ends up behind the section): for every layer the K rows [0, n_kv) then the V rows, in
 * the reference layout (src/q4_fwd.c:2353-2360 save, :2437-2445 restore).  Rows are converted on the
 * device and pass through pinned staging buffers; a seekable descriptor is written / read by several I/O
 * threads at once (pwrite / pread at precomputed offsets, $Q4_SESS_IO_THREADS), a pipe or socket in order.
 * Blocking; returns false on a short file or I/O error, and a regular file that is too short is refused
 * before any row is applied. */
bool q4_gpu_kv_write_fd(const q4_gpu_kv *kv, uint32_t n_kv, int fd);
bool q4_gpu_kv_read_fd(q4_gpu_kv *kv, uint32_t n_kv, int fd);

/* ---- the whole session file, format version 5 (q4_sess_save / q4_sess_restore / q4_sess_peek_ids and
 * q4_sess_hdr, src/q4_fwd.c:2256-2477, 2636-2657).  The store supplies the KV section and the header
 * fields it knows (max_kv, n_kv, number of attention layers, row width, KV kind tag); everything else is
 * the host's and travels through this descriptor: header fields, token ids, and the state sections as
 * opaque host bytes in file order.  A file written by q4_gpu_sess_file_write is byte for byte what the
 * reference host writes for the same state, and the other way round.
 *   state_a : last residual + PLE convolution state, 11 * hc_dim floats                  (:2345-2347)
 *   state_b : recurrent-layer state n_gdn*n_v_h*d_v*d_v floats + convolution history
 *             n_gdn*conv_hist*conv_ch floats                                             (:2357-2362)
 *   idx_raw : the indexer's fp16 raw keys, n_layers * n_kv * idx_dim * 2 bytes in layer order, or NULL
 *             (the file then records "no keys")                                          (:2363-2372)
 * The sizes must be exactly what the header dimensions imply, else the call is rejected. */
typedef struct q4_gpu_sess_desc {
    uint64_t bytes_total;                 /* model guard */
    uint32_t n_layer, n_expert;
    uint32_t pos;                         /* written from / restored into */
    uint32_t n_gdn, n_v_h, d_v, conv_hist, conv_ch, hc_dim;
    uint32_t prompt_n, nmsg;
    uint64_t user_hash;
    const int32_t *ids;                   /* write: the ids that produced the state; read: not used (see `ids` argument) */
    uint32_t n_ids;                       /* write: their count; read: set to the saved count */
    int32_t ple_hist[8];
    void *state_a;
    uint64_t state_a_bytes;
    void *state_b;
    uint64_t state_b_bytes;
    uint32_t idx_dim;
    uint32_t idx_has_raw;                 /* read: 1 if the file carried raw keys (copied to idx_raw) */
    void *idx_raw;
    uint64_t idx_raw_bytes;               /* write: exact size; read: capacity of idx_raw */
} q4_gpu_sess_desc;
/* Size of the file q4_gpu_sess_file_write would produce. */
uint64_t q4_gpu_sess_file_bytes(const q4_gpu_kv *kv, uint32_t n_kv, const q4_gpu_sess_desc *d);
/* q4_sess_save: writes "<path>.tmp" and renames it over path, so a reader never sees a torn file; on any
 * failure the temporary file is removed and false is returned. */
bool q4_gpu_sess_file_write(const q4_gpu_kv *kv, uint32_t n_kv, const q4_gpu_sess_desc *d, const char *path);
/* q4_sess_restore: returns the saved prefix length when the file is accepted (rows [0, n_kv) of every
 * layer restored into the store, state sections copied into the descriptor's buffers, pos / prompt_n / nmsg /
 * user_hash / ple_hist / n_ids set), else 0.  Accepted only if magic, version, model guard and every
 * dimension match, max_kv and the KV kind are those of the store (the rows are raw: :2405-2408), the file
 * holds exactly n_kv == n_ids rows, n_ids <= the caller's n_ids and every saved id equals ids[i] (exact
 * prefix: :2417-2432).  The file's length is checked before anything is applied; after a failure in the
 * middle of the KV section the store's rows are unspecified, as in the reference (which resets the session). */
int q4_gpu_sess_file_read(q4_gpu_kv *kv, q4_gpu_sess_desc *d, const int32_t *ids, int n_ids, const char *path);
/* q4_sess_peek_ids: the saved ids and prompt metadata without touching any state; -1 if the file is not a
 * version-5 session of this model (bytes_total, n_layer, n_expert of `model`) or holds more than max_ids. */
int q4_gpu_sess_file_peek_ids(const q4_gpu_sess_desc *model, const char *path, int32_t *ids, int max_ids,
                              uint32_t *prompt_n, uint32_t *nmsg, uint64_t *user_hash);

/* ---- decode attention over a store.  One launch covers every kv head and query head of the
 * layer (split-KV over the position list, merged by the last block to finish).
 *  q        : [n_head][hd], fp32 (q_bf16 = 0) or bf16 (q_bf16 = 1)
 *  gate     : [n_head][hd] fp32 or NULL (no gate)
 *  idx      : NULL = dense over [0, n_kv); else `width` int32 positions per list, -1 = skip;
 *             idx_kvh_stride = 0: one list shared by all kv heads (the reference), else the list
 *             of kv head kh starts at idx + kh*idx_kvh_stride (one list per kv head)
 *  n_kv     : rows attended in dense mode; in indexed mode the number of rows written so far: list
 *             entries >= n_kv are skipped and raise status bit 4 (the store is not cleared when it
 *             is created, so rows beyond n_kv hold nothing meaningful); 0 = take (device position
 *             word + 1), as the graph-captured reference path does
 *  out      : [n_head][hd] fp32
 * Replaces q4_hip_qsa_decode_idx / q4_hip_qsa_decode_n for n_tok = 1 (src/q4_fwd.c:738-741,922). */
bool q4_gpu_kv_decode(const q4_gpu_kv *kv, uint32_t layer, const void *q, int q_bf16,
                      const float *gate, float *out, uint32_t n_head, const int32_t *idx,
                      uint32_t width, uint32_t idx_kvh_stride, uint32_t n_kv, float scale);
/* ---- decode with no allocation at all.  Has no counterpart in the reference.  Same arguments and
 * result as q4_gpu_kv_decode, for hosts that may not allocate device memory once they are running: an
 * engine whose placement planner has already handed every byte of device memory to weights, expert
 * slots and KV (a late cudaMalloc can fail, and it synchronises the device), or a serving loop that
 * must never enter the allocator.  The split-KV records live in a 4 MB array inside the library
 * image (held by every GPU that loads the library until the process exits), so:
 *  - shapes are limited to 4 kv heads and 16 query heads per kv head; anything larger returns false
 *    with status bit 8; the number of splits shrinks automatically until the records fit;
 *  - the first call on a device looks up the array's device address (cudaGetSymbolAddress); make that
 *    first call during start-up, before any stream capture is opened;
 *  - every call shares the one array and keeps the previous call's contents: the arrival counters are
 *    cleared on the stream before each launch, and two calls that overlap on the GPU (different
 *    streams, or another process thread) race on it -- keep calls stream-ordered.
 * Calls no cudaMalloc / cudaFree and no allocating library routine. */
bool q4_gpu_kv_decode_noalloc(const q4_gpu_kv *kv, uint32_t layer, const void *q, int q_bf16,
                              const float *gate, float *out, uint32_t n_head, const int32_t *idx,
                              uint32_t width, uint32_t idx_kvh_stride, uint32_t n_kv, float scale);

/* Sparse prefill on the store: n_tok queries q [n_tok][n_head][hd], each attending the rows its own list
 * names, idx[t * idx_tok_stride + kv_head * idx_kvh_stride + j] (j < width, -1 = skip; idx_kvh_stride 0 =
 * one list per token shared by the kv heads, the reference's form); out [n_tok][n_head][hd], gate
 * likewise or NULL.  The n_tok > 1 case of q4_hip_qsa_decode_idx (src/q4.h:911-915; gqa_prefill_k<KIND,
 * true>, src/q4_rocm.cu:7319,7342-7357) on the library-owned store, one launch. */
bool q4_gpu_kv_decode_idx_n(const q4_gpu_kv *kv, uint32_t layer, const void *q, int q_bf16,
                            const float *gate, float *out, uint32_t n_head, const int32_t *idx,
                            uint32_t width, uint32_t idx_kvh_stride, uint32_t idx_tok_stride,
                            uint32_t n_tok, float scale);

/* Same, but stops before normalisation: part[n_head][hd+2] = {m, l, acc[hd]} over this store's
 * rows, the record of src/q4_rocm.cu:6780,6957-6963 -- the payload exchanged between GPUs when one
 * sequence is sharded by position. */
bool q4_gpu_kv_decode_partial(const q4_gpu_kv *kv, uint32_t layer, const void *q, int q_bf16,
                              float *part, uint32_t n_head, const int32_t *idx, uint32_t width,
                              uint32_t idx_kvh_stride, uint32_t n_kv, float scale);
/* Merge n_parts records per head (gqa_dec_comb_k, src/q4_rocm.cu:6968-7012):
 * parts [n_parts][n_head][hd+2] -> out [n_head][hd], times sigmoid(gate) when gate != NULL. */
bool q4_gpu_lse_merge(const float *parts, uint32_t n_parts, uint32_t n_head, uint32_t hd,
                      const float *gate, float *out);

/* ---- sequence-sharded decode with the exchange inside the kernel.  No counterpart in the reference
 * (it runs one GPU); the merge is gqa_dec_comb_k's (src/q4_rocm.cu:6968-7012), taken across GPUs.
 * Every rank of a node owns the rows [b, e) of one context in a store of its own and an exchange
 * window; q4_gpu_kv_decode_xchg attends the local rows, stores the rank's (acc, m, l) record into
 * every peer's window over NVLink (8-byte packets that carry the call's epoch, so no fence or flag
 * follows them), polls (bounded) for the peers' records in its own window and writes the merged,
 * gated output on every rank: one launch per layer, no host round trip, no collective library.
 *   create   : rank/world <= 16, n_kvh <= 16; allocates the window (cudaMalloc) and clears it.
 *   handle   : the 64-byte CUDA IPC handle of the local window, to be sent to every peer once.
 *   attach   : opens a peer's handle (another process on the same node, peer access required).
 *   attach_ptr: a peer window that is already mapped in this process (q4_gpu_xchg_window of an
 *              exchange object on the same device, or any mapping the host obtained itself).
 *   phase    : 0 = attend, push, wait and merge in one kernel; 1 = attend and push only; 2 = wait
 *              and merge only (kv, q, n_kv, scale ignored).  1 then 2 on every rank equals 0.
 *   Every rank must make the same sequence of calls.  A wait that outlasts the limit (2 s unless
 *   set) sets status bit 32 in q4_gpu_last_error() and the output is this rank's own part only; the
 *   context stays usable. */
typedef struct q4_gpu_xchg q4_gpu_xchg;
q4_gpu_xchg *q4_gpu_xchg_create(uint32_t rank, uint32_t world, uint32_t n_head, uint32_t n_kvh, uint32_t hd);
void q4_gpu_xchg_destroy(q4_gpu_xchg *x);
bool q4_gpu_xchg_handle(q4_gpu_xchg *x, void *handle64);
void *q4_gpu_xchg_window(q4_gpu_xchg *x);
bool q4_gpu_xchg_attach(q4_gpu_xchg *x, uint32_t peer_rank, const void *handle64);
bool q4_gpu_xchg_attach_ptr(q4_gpu_xchg *x, uint32_t peer_rank, void *peer_window);
bool q4_gpu_xchg_set_timeout_ms(q4_gpu_xchg *x, uint32_t ms);
bool q4_gpu_kv_decode_xchg(const q4_gpu_kv *kv, q4_gpu_xchg *x, uint32_t layer, const void *q, int q_bf16,
                           const float *gate, float *out, uint32_t n_kv, float scale, int phase);

/* ---- the same exchange as a collective: NCCL all-gather of the ranks' records + merge.  No counterpart in
 * the reference (one GPU, no collective); the merge is gqa_dec_comb_k's (src/q4_rocm.cu:6968-7012).  The
 * communicator comes from a 128-byte unique id made on one rank (q4_gpu_comm_unique_id) and handed to the
 * others by the host over any channel; one process per GPU.  NCCL is loaded at run time (libnccl.so.2, or
 * $Q4_NCCL_LIB): the library does not link it, and a host that never calls these never loads it.
 *   allgather_merge: part [n_head][hd+2] (from q4_gpu_kv_decode_partial) -> parts_all [world][n_head][hd+2]
 *   on every rank -> out [n_head][hd], times sigmoid(gate) when gate != NULL; enqueued on the compute
 *   stream (capturable in a graph like any NCCL call). */
typedef struct q4_gpu_comm q4_gpu_comm;
bool q4_gpu_comm_unique_id(void *id128);
q4_gpu_comm *q4_gpu_comm_create(const void *id128, uint32_t rank, uint32_t world);
void q4_gpu_comm_destroy(q4_gpu_comm *c);
bool q4_gpu_comm_allgather_merge(q4_gpu_comm *c, const float *part, float *parts_all, uint32_t n_head, uint32_t hd,
                                 const float *gate, float *out);

/* ---- batched multi-session decode: one launch per layer for every session of the batch. */
typedef struct q4_gpu_batch q4_gpu_batch;
q4_gpu_batch *q4_gpu_batch_create(uint32_t max_sessions);
void q4_gpu_batch_destroy(q4_gpu_batch *b);
/* Bind session slot s to a store (all stores of a batch share n_layers, n_kvh, hd and kind). */
bool q4_gpu_batch_bind(q4_gpu_batch *b, uint32_t slot, q4_gpu_kv *kv);
/* Publish the decode positions of sessions [0, n_sessions) (host array of n_sessions int32),
 * stream-ordered like q4_hip_pos_push.  n_sessions may be smaller than the number of bound slots: every
 * later q4_gpu_batch_append / _decode / _append_decode covers exactly these n_sessions sessions (their k,
 * v, q, gate, out and idx arrays have n_sessions rows) until the next call. */
bool q4_gpu_batch_set_pos(q4_gpu_batch *b, const int32_t *pos, uint32_t n_sessions);
/* pos[s] += delta on the device for the sessions of the last q4_gpu_batch_set_pos: stream-ordered and
 * capturable, so a decode step captured as one graph (advance by 1, then the layers) is replayed without a
 * host upload per step.  No counterpart in the reference (its graph reads one position word that the host
 * pushes every step, q4_hip_pos_push).  The dense split heuristic keeps using the largest position published
 * by set_pos (plus the advances made outside a capture). */
bool q4_gpu_batch_advance(q4_gpu_batch *b, int32_t delta);
/* k, v: [n_sessions][n_kvh*hd] fp32; row s goes to slot pos[s] of session s. */
bool q4_gpu_batch_append(q4_gpu_batch *b, uint32_t layer, const float *k, const float *v);
/* q [n_sessions][n_head][hd]; gate, out likewise; idx [n_sessions][...] with idx_sess_stride
 * entries between sessions (NULL = dense over [0, pos[s]+1)). */
bool q4_gpu_batch_decode(q4_gpu_batch *b, uint32_t layer, const void *q, int q_bf16,
                         const float *gate, float *out, const int32_t *idx, uint32_t width,
                         uint32_t idx_kvh_stride, uint32_t idx_sess_stride, uint32_t n_head,
                         float scale);
/* q4_gpu_batch_append then q4_gpu_batch_decode as one call; on a q8_0 store at hd 128 it is one launch per layer
 * (the attention kernel quantises and stores each session's newest K/V row itself, same bytes as the
 * append).  k, v: [n_sessions][n_kvh*hd] fp32.  Replaces the pair src/q4_fwd.c:891 + :922. */
bool q4_gpu_batch_append_decode(q4_gpu_batch *b, uint32_t layer, const float *k, const float *v, const void *q,
                                int q_bf16, const float *gate, float *out, const int32_t *idx, uint32_t width,
                                uint32_t idx_kvh_stride, uint32_t idx_sess_stride, uint32_t n_head, float scale);
/* Same for one session at the device position word (q4_gpu_kv_append_d + q4_gpu_kv_decode with n_kv = 0). */
bool q4_gpu_kv_append_decode_d(q4_gpu_kv *kv, uint32_t layer, const float *k, const float *v, const void *q,
                               int q_bf16, const float *gate, float *out, uint32_t n_head, const int32_t *idx,
                               uint32_t width, uint32_t idx_kvh_stride, float scale);

/* ---- dense causal prefill attention on the tensor cores (tcgen05 / TMEM): query t of the chunk
 * attends rows [0, kv_base + t + 1) of the store.  q, out: [n_tok][n_head][hd] bf16; gate: fp32 or
 * NULL.  Replaces q4_hip_qsa_decode_n with n_tok > 1 (gqa_prefill_k, src/q4_rocm.cu:7019-7206; host
 * slicing src/q4_fwd.c:1745-1753 is not needed). */
bool q4_gpu_kv_prefill(const q4_gpu_kv *kv, uint32_t layer, const void *q_bf16, const float *gate,
                       void *out_bf16, uint32_t n_head, uint32_t n_tok, uint32_t kv_base,
                       float scale);

#ifdef __cplusplus
}
#endif
#endif /* Q4_GPU_H */
