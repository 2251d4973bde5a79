/*
 * The session file of the reference host (q4_sess_save / q4_sess_restore / q4_sess_peek_ids,
 * src/q4_fwd.c:2256-2477, 2636-2657), format version 5, written and read around a library-owned KV store:
 *
 *   q4_sess_hdr (96 bytes) | token ids | PLE history (8 x int32) | residual + PLE convolution state
 *   | per attention layer: K rows [0, n_kv) then V rows, in the reference row layout
 *   | recurrent-layer state + convolution history | indexer meta (4 x uint32) | indexer raw keys
 *
 * The KV section comes from / goes to the store (rows converted on the device); the header fields the host
 * owns, the ids and the other state sections are the caller's, passed through as opaque bytes whose sizes
 * the header dimensions fix.  A file written here is what the reference host writes for the same state, and
 * the restore applies the reference's checks: magic, version, model guard, dimensions, max_kv and KV kind,
 * n_kv == n_ids, and an exact match of every saved id with the caller's prefix (:2405-2432).
 *
 * Data path of the KV section: export kernel -> device staging -> pinned host buffers (copy engine) ->
 * pwrite() at precomputed offsets from a few I/O threads, several chunks in flight; the reverse for reading
 * (pread into pinned buffers ahead of the uploads).  The reference does a synchronous 16 MiB device-to-host
 * copy + fwrite loop (:2276-2284).
 */
#include <errno.h>
#include <fcntl.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <mutex>
#include <thread>
#include <vector>

#include "q4_internal.h"

namespace {

constexpr uint32_t SESS_MAGIC = 0x53345134u;   /* "Q4SS", src/q4_fwd.c:2256 */
constexpr uint32_t SESS_VERSION = 5u;
constexpr size_t IO_CHUNK = (size_t)16 << 20;
constexpr int IO_BUFS = 8;

/* q4_sess_hdr, src/q4_fwd.c:2259-2271 (natural alignment: 96 bytes, user_hash at offset 88) */
struct SessHdr {
    uint32_t magic, version;
    uint64_t bytes_total;
    uint32_t n_layer, n_expert;
    uint32_t max_kv, n_kv, pos;
    uint32_t n_qsa, kvw;
    uint32_t n_gdn, n_v_h, d_v, conv_hist, conv_ch, hc_dim;
    uint32_t n_ids;
    uint32_t prompt_n;
    uint32_t nmsg;
    uint32_t pad;
    uint64_t user_hash;
};
static_assert(sizeof(SessHdr) == 96, "session header layout");

uint32_t kv_tag(int kind) { return kind == Q4K_Q8 ? 8u : kind == Q4K_F16 ? 2u : 4u; }   /* src/q4_fwd.c:663-665 */
uint32_t ref_token_bytes(const q4_gpu_kv *kv) {
    const uint32_t kvw = kv->n_kvh * kv->hd;
    return kv->kind == Q4K_Q8 ? kvw / 32u * 34u : kvw * (kv->kind == Q4K_F16 ? 2u : 4u);
}

bool pwrite_all(int fd, const uint8_t *p, size_t n, off_t off) {
    while (n) {
        ssize_t w = pwrite(fd, p, n, off);
        if (w < 0 && errno == EINTR) continue;
        if (w <= 0) return false;
        p += w; n -= (size_t)w; off += w;
    }
    return true;
}
bool pread_all(int fd, uint8_t *p, size_t n, off_t off) {
    while (n) {
        ssize_t r = pread(fd, p, n, off);
        if (r < 0 && errno == EINTR) continue;
        if (r <= 0) return false;   /* a short file fails here */
        p += r; n -= (size_t)r; off += r;
    }
    return true;
}
bool write_seq(int fd, const uint8_t *p, size_t n) {
    while (n) {
        ssize_t w = write(fd, p, n);
        if (w < 0 && errno == EINTR) continue;
        if (w <= 0) return false;
        p += w; n -= (size_t)w;
    }
    return true;
}
bool read_seq(int fd, uint8_t *p, size_t n) {
    while (n) {
        ssize_t r = read(fd, p, n);
        if (r < 0 && errno == EINTR) continue;
        if (r <= 0) return false;
        p += r; n -= (size_t)r;
    }
    return true;
}

/* staging buffers, allocated on first use and kept until shutdown (pinning memory costs milliseconds) */
struct Staging {
    uint8_t *dev = nullptr, *host[IO_BUFS] = {};
    cudaEvent_t ev[IO_BUFS] = {};
    bool ok = false;
} g_stage_io;

bool staging_get() {
    Staging &S = g_stage_io;
    if (S.ok) return true;
    bool ok = cudaMalloc(&S.dev, IO_BUFS * IO_CHUNK) == cudaSuccess;
    for (int i = 0; ok && i < IO_BUFS; i++)
        ok = cudaMallocHost(&S.host[i], IO_CHUNK) == cudaSuccess &&
             cudaEventCreateWithFlags(&S.ev[i], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
        (void)cudaGetLastError();
        return false;
    }
    S.ok = true;
    return true;
}

/* one chunk of the KV section: rows [t0, t0 + n) of K (which 0) or V (1) of a layer, at byte `off` of the section */
struct Chunk {
    uint32_t layer, t0, n;
    int which;
    uint64_t off;
};
std::vector<Chunk> kv_chunks(const q4_gpu_kv *kv, uint32_t n_kv) {
    std::vector<Chunk> c;
    const uint32_t tb = ref_token_bytes(kv), rows = (uint32_t)(IO_CHUNK / tb);
    uint64_t off = 0;
    for (uint32_t layer = 0; layer < kv->n_layers; layer++)
        for (int which = 0; which < 2; which++)
            for (uint32_t t0 = 0; t0 < n_kv; t0 += rows) {
                const uint32_t n = n_kv - t0 < rows ? n_kv - t0 : rows;
                c.push_back({layer, t0, n, which, off});
                off += (uint64_t)n * tb;
            }
    return c;
}
int io_threads() {
    unsigned hw = std::thread::hardware_concurrency();
    int n = hw >= 16 ? 6 : hw >= 8 ? 4 : 2;
    const char *e = getenv("Q4_SESS_IO_THREADS");
    if (e) n = atoi(e);
    return n < 1 ? 1 : n > IO_BUFS ? IO_BUFS : n;
}

/* A small in-order job board shared by the launching thread and the I/O threads: state[i] of chunk i goes
 * 0 (not issued) -> 1 (handed to the I/O threads) -> 2 (done). */
struct Board {
    std::mutex m;
    std::condition_variable cv;
    std::vector<int> state;
    size_t next = 0;      /* next chunk an I/O thread may take */
    bool failed = false;
};

/* KV section -> fd at [base, base + section bytes): seekable descriptors get parallel pwrite()s */
bool kv_section_write(const q4_gpu_kv *kv, uint32_t n_kv, int fd, off_t base, bool seekable) {
    if (!staging_get()) return q4i_fail(Q4E_CUDA, "session file: staging allocation failed");
    Staging &S = g_stage_io;
    const std::vector<Chunk> chunks = kv_chunks(kv, n_kv);
    const uint32_t tb = ref_token_bytes(kv);
    Board B;
    B.state.assign(chunks.size(), 0);
    /* Writes into one file serialise on its inode lock, so the I/O threads copy into a shared mapping of the
     * section instead (the file is grown to its final size first); a descriptor that cannot be mapped
     * (write-only, not a regular file) takes pwrite(). */
    const uint64_t total = chunks.empty() ? 0 : chunks.back().off + (uint64_t)chunks.back().n * tb;
    uint8_t *map = nullptr;
    size_t map_len = 0, map_skew = 0;
    if (seekable && total) {
        struct stat sb;
        const long pg = sysconf(_SC_PAGESIZE);
        if (fstat(fd, &sb) == 0 && (S_ISREG(sb.st_mode)) && pg > 0 &&
            (sb.st_size >= base + (off_t)total || ftruncate(fd, base + (off_t)total) == 0)) {
            map_skew = (size_t)(base % pg);
            map_len = (size_t)total + map_skew;
            void *m = mmap(nullptr, map_len, PROT_WRITE, MAP_SHARED, fd, base - (off_t)map_skew);
            if (m != MAP_FAILED) map = (uint8_t *)m;
        }
    }
    auto worker = [&]() {
        for (;;) {
            size_t i;
            {
                std::unique_lock<std::mutex> lk(B.m);
                B.cv.wait(lk, [&] { return B.failed || B.next >= chunks.size() || B.state[B.next] == 1; });
                if (B.failed || B.next >= chunks.size()) return;
                i = B.next++;
            }
            const int buf = (int)(i % IO_BUFS);
            bool ok = cudaEventSynchronize(S.ev[buf]) == cudaSuccess;
            if (ok && map) {
                /* the chunk's pages are brought into the mapping in one call (the kernel ignores the advice where
                 * it does not know it) instead of one fault per page under the copy: 11.8 against 6.9 GB/s with six
                 * threads on an in-memory file */
                uint8_t *dst = map + map_skew + chunks[i].off;
                const size_t len = (size_t)chunks[i].n * tb;
                const uintptr_t pg = (uintptr_t)sysconf(_SC_PAGESIZE);
                uint8_t *lo = (uint8_t *)((uintptr_t)dst & ~(pg - 1));
                (void)madvise(lo, (size_t)(dst + len - lo), 23 /* MADV_POPULATE_WRITE */);
                memcpy(dst, S.host[buf], len);
            }
            else if (ok) ok = pwrite_all(fd, S.host[buf], (size_t)chunks[i].n * tb, base + (off_t)chunks[i].off);
            {
                std::lock_guard<std::mutex> lk(B.m);
                B.state[i] = 2;
                if (!ok) B.failed = true;
            }
            B.cv.notify_all();
        }
    };
    std::vector<std::thread> pool;
    const int n_thr = seekable ? io_threads() : 1;
    if (seekable)
        for (int t = 0; t < n_thr; t++) pool.emplace_back(worker);
    bool ok = true;
    for (size_t i = 0; i < chunks.size() && ok; i++) {
        const int buf = (int)(i % IO_BUFS);
        if (i >= IO_BUFS) {   /* the buffer's previous chunk must be on its way to the file */
            if (seekable) {
                std::unique_lock<std::mutex> lk(B.m);
                B.cv.wait(lk, [&] { return B.failed || B.state[i - IO_BUFS] == 2; });
                if (B.failed) { ok = false; break; }
            }
        }
        uint8_t *stage = S.dev + (size_t)buf * IO_CHUNK;
        const Chunk &c = chunks[i];
        ok = q4_gpu_kv_export(kv, c.layer, c.which, c.t0, c.n, stage) &&
             cudaMemcpyAsync(S.host[buf], stage, (size_t)c.n * tb, cudaMemcpyDeviceToHost, g_q4.stream) == cudaSuccess &&
             cudaEventRecord(S.ev[buf], g_q4.stream) == cudaSuccess;
        if (!ok) break;
        if (seekable) {
            { std::lock_guard<std::mutex> lk(B.m); B.state[i] = 1; }
            B.cv.notify_all();
        } else {   /* a pipe or socket: in order, on this thread */
            ok = cudaEventSynchronize(S.ev[buf]) == cudaSuccess && write_seq(fd, S.host[buf], (size_t)c.n * tb);
        }
    }
    if (seekable) {
        {
            std::lock_guard<std::mutex> lk(B.m);
            if (!ok) B.failed = true;
        }
        B.cv.notify_all();
        {   /* wait for the chunks in flight, then let the threads go */
            std::unique_lock<std::mutex> lk(B.m);
            B.cv.wait(lk, [&] {
                if (B.failed) return true;
                for (int st : B.state) if (st != 2) return false;
                return true;
            });
            if (B.failed) ok = false;
            B.next = chunks.size();
        }
        B.cv.notify_all();
        for (auto &t : pool) t.join();
    }
    if (map) munmap(map, map_len);
    (void)cudaStreamSynchronize(g_q4.stream);
    return ok;
}

/* fd [base, ..) -> KV section of the store: pread()s run ahead of the uploads on the I/O threads */
bool kv_section_read(q4_gpu_kv *kv, uint32_t n_kv, int fd, off_t base, bool seekable) {
    if (!staging_get()) return q4i_fail(Q4E_CUDA, "session file: staging allocation failed");
    Staging &S = g_stage_io;
    const std::vector<Chunk> chunks = kv_chunks(kv, n_kv);
    const uint32_t tb = ref_token_bytes(kv);
    /* state: 0 = buffer not free yet, 1 = may be read into, 2 = read done, 3 = read failed */
    Board B;
    B.state.assign(chunks.size(), 0);
    for (size_t i = 0; i < chunks.size() && i < (size_t)IO_BUFS; i++) B.state[i] = 1;
    auto worker = [&]() {
        for (;;) {
            size_t i;
            {
                std::unique_lock<std::mutex> lk(B.m);
                B.cv.wait(lk, [&] { return B.failed || B.next >= chunks.size() || B.state[B.next] == 1; });
                if (B.failed || B.next >= chunks.size()) return;
                i = B.next++;
            }
            const bool ok = pread_all(fd, S.host[i % IO_BUFS], (size_t)chunks[i].n * tb, base + (off_t)chunks[i].off);
            {
                std::lock_guard<std::mutex> lk(B.m);
                B.state[i] = ok ? 2 : 3;
                if (!ok) B.failed = true;
            }
            B.cv.notify_all();
        }
    };
    std::vector<std::thread> pool;
    if (seekable)
        for (int t = 0; t < io_threads(); t++) pool.emplace_back(worker);
    bool ok = true;
    for (size_t i = 0; i < chunks.size() && ok; i++) {
        const int buf = (int)(i % IO_BUFS);
        const Chunk &c = chunks[i];
        if (seekable) {
            std::unique_lock<std::mutex> lk(B.m);
            B.cv.wait(lk, [&] { return B.state[i] >= 2 || B.failed; });
            if (B.state[i] != 2) { ok = false; break; }
        } else {
            if (i >= (size_t)IO_BUFS && cudaEventSynchronize(S.ev[buf]) != cudaSuccess) { ok = false; break; }
            if (!read_seq(fd, S.host[buf], (size_t)c.n * tb)) { ok = false; break; }
        }
        uint8_t *stage = S.dev + (size_t)buf * IO_CHUNK;
        ok = cudaMemcpyAsync(stage, S.host[buf], (size_t)c.n * tb, cudaMemcpyHostToDevice, g_q4.stream) == cudaSuccess &&
             q4_gpu_kv_import(kv, c.layer, c.which, c.t0, c.n, stage) &&
             cudaEventRecord(S.ev[buf], g_q4.stream) == cudaSuccess;
        if (ok && seekable && i + IO_BUFS < chunks.size()) {
            /* the buffer may take the chunk IO_BUFS ahead once this upload has left it */
            ok = cudaEventSynchronize(S.ev[buf]) == cudaSuccess;
            { std::lock_guard<std::mutex> lk(B.m); B.state[i + IO_BUFS] = 1; }
            B.cv.notify_all();
        }
    }
    if (seekable) {
        {
            std::lock_guard<std::mutex> lk(B.m);
            if (!ok) B.failed = true;
            B.next = ok ? B.next : chunks.size();
        }
        B.cv.notify_all();
        for (auto &t : pool) t.join();
    }
    (void)cudaStreamSynchronize(g_q4.stream);
    return ok;
}

bool is_seekable(int fd, off_t *pos) {
    const off_t p = lseek(fd, 0, SEEK_CUR);
    if (p == (off_t)-1) return false;
    *pos = p;
    return true;
}

uint64_t state_a_bytes(uint32_t hc_dim) { return 11ull * hc_dim * sizeof(float); }   /* residual + 10 x hc_dim PLE convolution */
uint64_t state_b_bytes(const q4_gpu_sess_desc *d) {
    return ((uint64_t)d->n_gdn * d->n_v_h * d->d_v * d->d_v + (uint64_t)d->n_gdn * d->conv_hist * d->conv_ch) * sizeof(float);
}

}  // namespace

void q4i_sess_release() {
    Staging &S = g_stage_io;
    if (S.dev) cudaFree(S.dev);
    for (int i = 0; i < IO_BUFS; i++) {
        if (S.host[i]) cudaFreeHost(S.host[i]);
        if (S.ev[i]) cudaEventDestroy(S.ev[i]);
    }
    S = Staging();
}

/* The KV section alone, at the descriptor's current position (advanced past it on return). */
extern "C" bool q4_gpu_kv_write_fd(const q4_gpu_kv *kv, uint32_t n_kv, int fd) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "kv_write_fd: library not initialised");
    Q4_REQUIRE(kv && n_kv && n_kv <= kv->max_kv && fd >= 0 && !g_q4.capturing, "kv_write_fd: bad argument");
    off_t base = 0;
    const bool seekable = is_seekable(fd, &base);
    const uint64_t total = (uint64_t)kv->n_layers * 2ull * n_kv * ref_token_bytes(kv);
    if (!kv_section_write(kv, n_kv, fd, base, seekable)) return q4i_fail(Q4E_CUDA, "kv_write_fd: copy or write failed");
    if (seekable && lseek(fd, base + (off_t)total, SEEK_SET) == (off_t)-1) return q4i_fail(Q4E_CUDA, "kv_write_fd: seek failed");
    return true;
}
extern "C" bool q4_gpu_kv_read_fd(q4_gpu_kv *kv, uint32_t n_kv, int fd) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "kv_read_fd: library not initialised");
    Q4_REQUIRE(kv && n_kv && n_kv <= kv->max_kv && fd >= 0 && !g_q4.capturing, "kv_read_fd: bad argument");
    off_t base = 0;
    const bool seekable = is_seekable(fd, &base);
    const uint64_t total = (uint64_t)kv->n_layers * 2ull * n_kv * ref_token_bytes(kv);
    if (seekable) {   /* a short file is refused before anything is applied */
        struct stat sb;
        if (fstat(fd, &sb) == 0 && S_ISREG(sb.st_mode) && (uint64_t)sb.st_size < (uint64_t)base + total)
            return q4i_fail(Q4E_ARG, "kv_read_fd: file shorter than the KV section");
    }
    if (!kv_section_read(kv, n_kv, fd, base, seekable)) return q4i_fail(Q4E_CUDA, "kv_read_fd: short file, read error or copy failure");
    if (seekable && lseek(fd, base + (off_t)total, SEEK_SET) == (off_t)-1) return q4i_fail(Q4E_CUDA, "kv_read_fd: seek failed");
    return true;
}

extern "C" uint64_t q4_gpu_sess_file_bytes(const q4_gpu_kv *kv, uint32_t n_kv, const q4_gpu_sess_desc *d) {
    if (!kv || !d) return 0;
    uint64_t n = sizeof(SessHdr) + (uint64_t)d->n_ids * 4 + 32 + state_a_bytes(d->hc_dim) +
                 (uint64_t)kv->n_layers * 2ull * n_kv * ref_token_bytes(kv) + state_b_bytes(d) + 16;
    if (d->idx_raw && d->idx_dim) n += (uint64_t)kv->n_layers * n_kv * d->idx_dim * 2;
    return n;
}

extern "C" bool q4_gpu_sess_file_write(const q4_gpu_kv *kv, uint32_t n_kv, const q4_gpu_sess_desc *d, const char *path) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "sess_file_write: library not initialised");
    Q4_REQUIRE(kv && d && path && n_kv && n_kv <= kv->max_kv && !g_q4.capturing, "sess_file_write: bad argument");
    Q4_REQUIRE(d->ids && d->n_ids > 0, "sess_file_write: no token ids");
    Q4_REQUIRE(d->state_a_bytes == state_a_bytes(d->hc_dim) && (d->state_a || !d->state_a_bytes),
               "sess_file_write: residual / PLE state must be 11 * hc_dim floats");
    Q4_REQUIRE(d->state_b_bytes == state_b_bytes(d) && (d->state_b || !d->state_b_bytes),
               "sess_file_write: recurrent state size does not follow from n_gdn, n_v_h, d_v, conv_hist, conv_ch");
    const uint64_t raw_bytes = d->idx_raw && d->idx_dim ? (uint64_t)kv->n_layers * n_kv * d->idx_dim * 2 : 0;
    Q4_REQUIRE(d->idx_raw_bytes == raw_bytes, "sess_file_write: indexer key bytes must be n_layers * n_kv * idx_dim * 2");
    SessHdr h;
    memset(&h, 0, sizeof(h));
    h.magic = SESS_MAGIC; h.version = SESS_VERSION; h.bytes_total = d->bytes_total;
    h.n_layer = d->n_layer; h.n_expert = d->n_expert;
    h.max_kv = kv->max_kv; h.n_kv = n_kv; h.pos = d->pos;
    h.n_qsa = kv->n_layers; h.kvw = kv->n_kvh * kv->hd;
    h.n_gdn = d->n_gdn; h.n_v_h = d->n_v_h; h.d_v = d->d_v; h.conv_hist = d->conv_hist; h.conv_ch = d->conv_ch;
    h.hc_dim = d->hc_dim;
    h.n_ids = d->n_ids;
    h.prompt_n = d->prompt_n > d->n_ids ? d->n_ids : d->prompt_n;   /* :2317-2318 */
    h.nmsg = d->nmsg;
    h.pad = kv_tag(kv->kind);
    h.user_hash = d->user_hash;
    char tmp[4096 + 16];
    if (strlen(path) > 4096) return q4i_fail(Q4E_ARG, "sess_file_write: path too long");
    snprintf(tmp, sizeof(tmp), "%s.tmp", path);
    const int fd = open(tmp, O_RDWR | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) return q4i_fail(Q4E_ARG, "sess_file_write: cannot create the temporary file");
    off_t off = 0;
    auto put = [&](const void *p, uint64_t n) {
        if (!n) return true;
        if (!pwrite_all(fd, (const uint8_t *)p, (size_t)n, off)) return false;
        off += (off_t)n;
        return true;
    };
    bool ok = put(&h, sizeof(h)) && put(d->ids, (uint64_t)d->n_ids * 4) && put(d->ple_hist, 32) &&
              put(d->state_a, d->state_a_bytes);
    if (ok) {
        ok = kv_section_write(kv, n_kv, fd, off, true);
        off += (off_t)((uint64_t)kv->n_layers * 2ull * n_kv * ref_token_bytes(kv));
    }
    if (ok) ok = put(d->state_b, d->state_b_bytes);
    if (ok) {
        const uint32_t meta[4] = {d->idx_dim, kv->n_layers, n_kv, raw_bytes ? 1u : 0u};   /* :2364 */
        ok = put(meta, sizeof(meta)) && put(d->idx_raw, raw_bytes);
    }
    if (close(fd) != 0) ok = false;
    if (!ok || rename(tmp, path) != 0) {
        unlink(tmp);
        return q4i_fail(Q4E_CUDA, "sess_file_write: write failed; no file was left behind");
    }
    return true;
}

/* reads and checks the header and the ids; on success the file position data is returned through *hdr */
static int open_checked(const char *path, const q4_gpu_sess_desc *want, bool model_guard_only, SessHdr *hdr) {
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return -1;
    if (!pread_all(fd, (uint8_t *)hdr, sizeof(*hdr), 0) || hdr->magic != SESS_MAGIC || hdr->version != SESS_VERSION ||
        hdr->bytes_total != want->bytes_total || hdr->n_layer != want->n_layer || hdr->n_expert != want->n_expert ||
        hdr->n_ids == 0) {
        close(fd);
        return -1;
    }
    (void)model_guard_only;
    return fd;
}

extern "C" int q4_gpu_sess_file_peek_ids(const q4_gpu_sess_desc *model, const char *path, int32_t *ids, int max_ids,
                                         uint32_t *prompt_n, uint32_t *nmsg, uint64_t *user_hash) {
    if (prompt_n) *prompt_n = 0;
    if (nmsg) *nmsg = 0;
    if (user_hash) *user_hash = 0;
    if (!model || !path || !ids || max_ids <= 0) return -1;
    SessHdr h;
    const int fd = open_checked(path, model, true, &h);
    if (fd < 0) return -1;
    bool ok = (int64_t)h.n_ids <= (int64_t)max_ids && h.prompt_n <= h.n_ids &&
              pread_all(fd, (uint8_t *)ids, (size_t)h.n_ids * 4, sizeof(SessHdr));
    close(fd);
    if (!ok) return -1;
    if (prompt_n) *prompt_n = h.prompt_n;
    if (nmsg) *nmsg = h.nmsg;
    if (user_hash) *user_hash = h.user_hash;
    return (int)h.n_ids;
}

extern "C" int q4_gpu_sess_file_read(q4_gpu_kv *kv, q4_gpu_sess_desc *d, const int32_t *ids, int n_ids, const char *path) {
    if (!g_q4.ok) { q4i_fail(Q4E_INIT, "sess_file_read: library not initialised"); return 0; }
    if (!kv || !d || !ids || n_ids <= 0 || !path || g_q4.capturing) { q4i_fail(Q4E_ARG, "sess_file_read: bad argument"); return 0; }
    SessHdr h;
    const int fd = open_checked(path, d, false, &h);
    if (fd < 0) return 0;
    /* the reference's acceptance test, src/q4_fwd.c:2405-2416: same model, same dimensions, same capacity and
     * KV kind (the rows are stored raw), a snapshot of exactly its ids, not longer than the caller's sequence */
    bool ok = h.max_kv == kv->max_kv && h.n_qsa == kv->n_layers && h.n_gdn == d->n_gdn && h.kvw == kv->n_kvh * kv->hd &&
              h.conv_ch == d->conv_ch && h.conv_hist == d->conv_hist && h.n_v_h == d->n_v_h && h.d_v == d->d_v &&
              h.hc_dim == d->hc_dim && h.pad == kv_tag(kv->kind) && h.n_kv == h.n_ids && (int64_t)h.n_ids <= (int64_t)n_ids &&
              h.n_kv <= kv->max_kv;
    ok = ok && d->state_a_bytes == state_a_bytes(h.hc_dim) && (d->state_a || !d->state_a_bytes) &&
         d->state_b_bytes == state_b_bytes(d) && (d->state_b || !d->state_b_bytes);
    off_t off = sizeof(SessHdr);
    if (ok) {   /* every saved id must equal the caller's: the state exists only at the end of the saved sequence */
        std::vector<int32_t> saved(h.n_ids);
        ok = pread_all(fd, (uint8_t *)saved.data(), (size_t)h.n_ids * 4, off);
        for (uint32_t i = 0; ok && i < h.n_ids; i++)
            if (saved[i] != ids[i]) {
                fprintf(stderr, "q4 gpu: session file prefix differs at token %u/%u (saved %d new %d)\n", i, h.n_ids,
                        saved[i], ids[i]);
                ok = false;
            }
        off += (off_t)h.n_ids * 4;
    }
    const uint64_t kv_bytes = (uint64_t)kv->n_layers * 2ull * h.n_kv * ref_token_bytes(kv);
    uint32_t meta[4] = {0, 0, 0, 0};
    int32_t ple[8];
    if (ok) {   /* the whole file must be there before anything is applied */
        struct stat sb;
        const off_t meta_off = off + 32 + (off_t)d->state_a_bytes + (off_t)kv_bytes + (off_t)d->state_b_bytes;
        ok = fstat(fd, &sb) == 0 && sb.st_size >= meta_off + 16 && pread_all(fd, (uint8_t *)meta, 16, meta_off);
        if (ok && meta[3]) {
            const uint64_t raw = (uint64_t)kv->n_layers * h.n_kv * meta[0] * 2;
            ok = d->idx_raw && meta[0] == d->idx_dim && meta[1] == kv->n_layers && meta[2] == h.n_kv &&   /* :2452-2454 */
                 d->idx_raw_bytes >= raw && (uint64_t)sb.st_size >= (uint64_t)meta_off + 16 + raw &&
                 pread_all(fd, (uint8_t *)d->idx_raw, (size_t)raw, meta_off + 16);
        }
    }
    if (ok) ok = pread_all(fd, (uint8_t *)ple, 32, off);
    off += 32;
    if (ok && d->state_a_bytes) ok = pread_all(fd, (uint8_t *)d->state_a, (size_t)d->state_a_bytes, off);
    off += (off_t)d->state_a_bytes;
    if (ok) ok = kv_section_read(kv, h.n_kv, fd, off, true);
    off += (off_t)kv_bytes;
    if (ok && d->state_b_bytes) ok = pread_all(fd, (uint8_t *)d->state_b, (size_t)d->state_b_bytes, off);
    close(fd);
    if (!ok) return 0;
    memcpy(d->ple_hist, ple, 32);
    d->pos = h.pos;
    d->prompt_n = h.prompt_n;
    d->nmsg = h.nmsg;
    d->user_hash = h.user_hash;
    d->n_ids = h.n_ids;
    d->idx_has_raw = meta[3];
    return (int)h.n_ids;
}
