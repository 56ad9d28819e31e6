/* Prequantised-weight sidecar: the final quantised tensors of a checkpoint, stored once so that
 * later starts upload them instead of running the load-time quantisers again.
 *
 * Contract: include/s2pro/qcache.h:34-54 of the reference.  The FILE is interchangeable with the
 * reference's, so its layout and staleness rule are given (src/sched/qcache.c:3-17, 74-113):
 *
 *   "S2PQC\1\0\0" | u64 fingerprint | u32 n | u32 0
 *   n x { u32 name_len, u32 kind, i32 N, i32 K, i32 group, u32 0,
 *         u64 q_off, u64 q_len, u64 s_off, u64 s_len, name bytes }
 *   payloads at 256-byte aligned absolute offsets
 *   kind 1: i8[N,K] + f32[N]; 2: nibbles[N,K/2] + f16[N*K/G]; 3: i8[N,K] + f16[N*K/G]
 *
 *   fingerprint = FNV-1a over "v1|mode=..|int4=..|g=..|mse=..|pk=..|all=.." and then, for every
 *   *.safetensors of the model directory in name order, its name, st_size and st_mtime.
 *
 * How this implementation works (its own, not the reference's):
 *  - reading: the sidecar is mapped (mmap) rather than read, its entry table is validated in one
 *    pass into a name-sorted index, and the mapping is registered with the CUDA driver as pinned
 *    memory, so the uploads of all tensors are queued back to back on the stream and overlap with
 *    whatever the loader does next; a tensor's lengths are checked against its shape before
 *    anything is allocated for it; nothing is copied on the host;
 *  - writing: quantised tensors are downloaded into one growing arena as they are put, and the
 *    file is produced at the end with a single positional write per region into a temporary
 *    that is renamed over the target (a reader never sees a half-written sidecar).
 * A mismatch or any problem on the reading side is a "miss": the live quantisers run.
 * S2P_QCACHE=0 disables the sidecar, S2P_QCACHE_DIR moves it.
 */
#include <dirent.h>
#include <errno.h>
#include <fcntl.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include "internal.h"

enum { QC_MAX_ENTRIES = 512, QC_HEADER_BYTES = 24, QC_ENTRY_BYTES = 56, QC_MAX_NAME = 512, QC_ALIGN = 256 };
static const char QC_MAGIC[8] = {'S', '2', 'P', 'Q', 'C', 1, 0, 0};

/* one tensor pair of the sidecar: where it is (file offsets when reading, arena offsets when writing) */
typedef struct {
    char* name;
    uint32_t kind;
    int32_t N, K, group;
    uint64_t q_off, q_len, s_off, s_len;
} qc_entry;

struct s2p_qcache {
    char path[1100];
    uint64_t fingerprint;
    int reading;
    qc_entry* entries; /* reading: sorted by name */
    int n, cap;
    /* reading */
    unsigned char* map;
    size_t map_len;
    int map_pinned;
    /* writing */
    unsigned char* arena;
    size_t arena_len, arena_cap;
};

/* ---- fingerprint ------------------------------------------------------------------------- */

static uint64_t fnv1a(uint64_t h, const void* data, size_t len) {
    for (const unsigned char* p = (const unsigned char*)data; len; len--) h = (h ^ *p++) * 0x100000001b3ULL;
    return h;
}
static int env_flag(const char* name, int unset_value) {
    const char* v = getenv(name);
    if (!v || !v[0]) return unset_value;
    return v[0] == '1' && !v[1];
}
static int is_shard(const struct dirent* de) {
    const size_t len = strlen(de->d_name);
    return len > 12 && strcmp(de->d_name + len - 12, ".safetensors") == 0;
}
static int by_byte_order(const struct dirent** a, const struct dirent** b) { return strcmp((*a)->d_name, (*b)->d_name); }

static int model_fingerprint(const char* dir, s2p_gemm_mode mode, uint64_t* out) {
    struct dirent** shards = NULL;
    const int n = scandir(dir, &shards, is_shard, by_byte_order);
    if (n <= 0) { free(shards); return 0; }
    char settings[256];
    const char* group = getenv("S2P_INT4_GROUP");
    snprintf(settings, sizeof(settings), "v1|mode=%d|int4=%d|g=%s|mse=%d|pk=%d|all=%d", (int)mode, env_flag("S2P_INT4", 0),
             group ? group : "32", env_flag("S2P_INT4_MSE", 1), env_flag("S2P_INT4_PACKED", 1), env_flag("S2P_INT4_ALL", 0));
    uint64_t h = fnv1a(0xcbf29ce484222325ULL, settings, strlen(settings));
    for (int i = 0; i < n; i++) {
        char full[1400];
        struct stat sb;
        snprintf(full, sizeof(full), "%s/%s", dir, shards[i]->d_name);
        if (stat(full, &sb) == 0) {
            h = fnv1a(h, shards[i]->d_name, strlen(shards[i]->d_name));
            h = fnv1a(h, &sb.st_size, sizeof(sb.st_size));
            h = fnv1a(h, &sb.st_mtime, sizeof(sb.st_mtime));
        }
        free(shards[i]);
    }
    free(shards);
    *out = h;
    return 1;
}

/* ---- reading ------------------------------------------------------------------------------- */

static uint32_t le32(const unsigned char* p) { uint32_t v; memcpy(&v, p, 4); return v; }
static uint64_t le64(const unsigned char* p) { uint64_t v; memcpy(&v, p, 8); return v; }
static int entry_by_name(const void* a, const void* b) { return strcmp(((const qc_entry*)a)->name, ((const qc_entry*)b)->name); }

static void drop_entries(s2p_qcache* qc) {
    for (int i = 0; i < qc->n; i++) free(qc->entries[i].name);
    free(qc->entries);
    qc->entries = NULL;
    qc->n = qc->cap = 0;
}
static void unmap_file(s2p_qcache* qc) {
    if (!qc->map) return;
    if (qc->map_pinned) cudaHostUnregister(qc->map);
    munmap(qc->map, qc->map_len);
    qc->map = NULL;
    qc->map_len = 0;
    qc->map_pinned = 0;
}

/* bytes a tensor pair of this kind and shape must have; 0 if the description is not one the library serves */
static int expected_lengths(uint32_t kind, int64_t N, int64_t K, int64_t group, uint64_t* q_len, uint64_t* s_len) {
    if (N <= 0 || K <= 0 || kind < 1 || kind > 3) return 0;
    if (kind == 1) { *q_len = (uint64_t)(N * K); *s_len = (uint64_t)N * 4; return 1; }
    if (group <= 0 || K % group || (kind == 2 && (K & 1))) return 0;
    *q_len = (uint64_t)(kind == 2 ? N * K / 2 : N * K);
    *s_len = (uint64_t)(N * (K / group)) * 2;
    return 1;
}

/* Map and index an existing sidecar; on anything unexpected the handle stays in write mode. */
static void open_for_reading(s2p_qcache* qc) {
    const int fd = open(qc->path, O_RDONLY);
    if (fd < 0) return;
    struct stat sb;
    if (fstat(fd, &sb) != 0 || sb.st_size < QC_HEADER_BYTES) { close(fd); return; }
    unsigned char* map = (unsigned char*)mmap(NULL, (size_t)sb.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) return;
    qc->map = map;
    qc->map_len = (size_t)sb.st_size;
    const uint64_t size = (uint64_t)sb.st_size;
    int good = memcmp(map, QC_MAGIC, 8) == 0;
    if (good && le64(map + 8) != qc->fingerprint) {
        fprintf(stderr, "[s2pro] qcache: stale fingerprint, rebuilding\n");
        good = 0;
    }
    const uint32_t n = good ? le32(map + 16) : 0;
    good = good && n >= 1 && n <= QC_MAX_ENTRIES;
    if (good) {
        qc->entries = (qc_entry*)calloc(n, sizeof(qc_entry));
        qc->cap = (int)n;
        good = qc->entries != NULL;
    }
    uint64_t at = QC_HEADER_BYTES;
    for (uint32_t i = 0; good && i < n; i++) {
        if (at + QC_ENTRY_BYTES > size) { good = 0; break; }
        const unsigned char* rec = map + at;
        qc_entry* e = &qc->entries[qc->n];
        const uint32_t name_len = le32(rec);
        e->kind = le32(rec + 4);
        e->N = (int32_t)le32(rec + 8);
        e->K = (int32_t)le32(rec + 12);
        e->group = (int32_t)le32(rec + 16);
        e->q_off = le64(rec + 24); e->q_len = le64(rec + 32);
        e->s_off = le64(rec + 40); e->s_len = le64(rec + 48);
        at += QC_ENTRY_BYTES;
        if (!name_len || name_len > QC_MAX_NAME || at + name_len > size) { good = 0; break; }
        /* the payload regions must lie inside the file (written without overflow: lengths first) */
        if (e->q_len > size || e->q_off > size - e->q_len || e->s_len > size || e->s_off > size - e->s_len) { good = 0; break; }
        e->name = (char*)malloc((size_t)name_len + 1);
        if (!e->name) { good = 0; break; }
        memcpy(e->name, map + at, name_len);
        e->name[name_len] = 0;
        at += name_len;
        qc->n++;
    }
    if (!good) {
        drop_entries(qc);
        unmap_file(qc);
        return;
    }
    qsort(qc->entries, (size_t)qc->n, sizeof(qc_entry), entry_by_name);
    /* pinned: cudaMemcpyAsync from the mapping is then a real asynchronous copy, so the uploads of all
     * tensors queue up behind one another while the loader goes on; without it the copies still work */
    qc->map_pinned = cudaHostRegister(qc->map, qc->map_len, cudaHostRegisterReadOnly) == cudaSuccess;
    if (!qc->map_pinned) cudaGetLastError(); /* clear the sticky-free error of a refused registration */
    qc->reading = 1;
}

s2p_status s2p_qcache_open(const char* model_dir, s2p_gemm_mode mode, s2p_qcache** out) {
    if (!model_dir || !out) return S2P_ERR_INVALID;
    *out = NULL;
    if (mode != S2P_GEMM_INT8 || !env_flag("S2P_QCACHE", 1)) return S2P_OK;
    uint64_t fp = 0;
    if (!model_fingerprint(model_dir, mode, &fp)) return S2P_OK;
    s2p_qcache* qc = (s2p_qcache*)calloc(1, sizeof(*qc));
    if (!qc) return S2P_ERR_OOM;
    qc->fingerprint = fp;
    const char* where = getenv("S2P_QCACHE_DIR");
    snprintf(qc->path, sizeof(qc->path), "%s/s2p_qcache.bin", (where && where[0]) ? where : model_dir);
    open_for_reading(qc);
    if (qc->reading) fprintf(stderr, "[s2pro] qcache: serving %d tensors from %s\n", qc->n, qc->path);
    else fprintf(stderr, "[s2pro] qcache: will write %s after load\n", qc->path);
    *out = qc;
    return S2P_OK;
}

int s2p_qcache_reading(const s2p_qcache* qc) { return qc && qc->reading; }

int s2p_qcache_try_load(s2p_qcache* qc, const char* name, int in_features, int out_features, s2p_linear* lin,
                        cudaStream_t stream) {
    if (!qc || !qc->reading || !name || !lin) return 0;
    qc_entry key;
    key.name = (char*)name;
    const qc_entry* e = (const qc_entry*)bsearch(&key, qc->entries, (size_t)qc->n, sizeof(qc_entry), entry_by_name);
    if (!e) {
        fprintf(stderr, "[s2pro] qcache: miss for %s (live path)\n", name);
        return 0;
    }
    uint64_t q_len = 0, s_len = 0;
    if (e->N != out_features || e->K != in_features || !expected_lengths(e->kind, e->N, e->K, e->group, &q_len, &s_len) ||
        q_len != e->q_len || s_len != e->s_len) {
        fprintf(stderr, "[s2pro] qcache: shape mismatch for %s\n", name);
        return 0;
    }
    s2p_linear fresh;
    memset(&fresh, 0, sizeof(fresh));
    fresh.in_features = in_features;
    fresh.out_features = out_features;
    s2p_tensor* codes = e->kind == 2 ? &fresh.w_pack : &fresh.w_int8;
    const int64_t code_shape[2] = {e->N, e->kind == 2 ? e->K / 2 : e->K};
    const int64_t scale_shape[1] = {e->kind == 1 ? (int64_t)e->N : (int64_t)e->N * (e->K / e->group)};
    int ok = s2p_tensor_device_alloc(codes, S2P_DT_I8, 2, code_shape) == S2P_OK &&
             s2p_tensor_device_alloc(&fresh.w_iscale, e->kind == 1 ? S2P_DT_F32 : S2P_DT_F16, 1, scale_shape) == S2P_OK;
    ok = ok && s2p_tensor_upload(codes, qc->map + e->q_off, e->q_len, stream) == S2P_OK &&
         s2p_tensor_upload(&fresh.w_iscale, qc->map + e->s_off, e->s_len, stream) == S2P_OK;
    if (!ok) {
        s2p_tensor_free(codes);
        s2p_tensor_free(&fresh.w_iscale);
        memset(lin, 0, sizeof(*lin));
        lin->in_features = in_features;
        lin->out_features = out_features;
        return 0;
    }
    fresh.int8_ready = 1;
    fresh.q_group = e->kind == 1 ? 0 : e->group;
    fresh.q_packed = e->kind == 2;
    *lin = fresh;
    return 1;
}

/* ---- writing ------------------------------------------------------------------------------- */

static unsigned char* arena_take(s2p_qcache* qc, size_t bytes, uint64_t* off) {
    if (qc->arena_len + bytes > qc->arena_cap) {
        size_t cap = qc->arena_cap ? qc->arena_cap : ((size_t)64 << 20);
        while (cap < qc->arena_len + bytes) cap *= 2;
        unsigned char* grown = (unsigned char*)realloc(qc->arena, cap);
        if (!grown) return NULL;
        qc->arena = grown;
        qc->arena_cap = cap;
    }
    *off = qc->arena_len;
    qc->arena_len += bytes;
    return qc->arena + *off;
}

s2p_status s2p_qcache_put_linear(s2p_qcache* qc, const char* name, const s2p_linear* lin, cudaStream_t stream) {
    /* the sidecar is an optimisation: whatever goes wrong here, the load itself goes on */
    if (!qc || qc->reading || !name || !lin || !lin->int8_ready || qc->n >= QC_MAX_ENTRIES) return S2P_OK;
    const s2p_tensor* codes = lin->q_packed ? &lin->w_pack : &lin->w_int8;
    if (!codes->data || !lin->w_iscale.data || strlen(name) > QC_MAX_NAME) return S2P_OK;
    if (qc->n == qc->cap) {
        const int cap = qc->cap ? qc->cap * 2 : 64;
        qc_entry* grown = (qc_entry*)realloc(qc->entries, (size_t)cap * sizeof(qc_entry));
        if (!grown) return S2P_OK;
        qc->entries = grown;
        qc->cap = cap;
    }
    qc_entry e;
    memset(&e, 0, sizeof(e));
    e.kind = lin->q_packed ? 2u : (lin->q_group > 0 ? 3u : 1u);
    e.N = lin->out_features;
    e.K = lin->in_features;
    e.group = lin->q_group;
    e.q_len = codes->bytes;
    e.s_len = lin->w_iscale.bytes;
    const size_t before = qc->arena_len;
    if (!arena_take(qc, codes->bytes, &e.q_off) || !arena_take(qc, lin->w_iscale.bytes, &e.s_off) || !(e.name = strdup(name))) {
        qc->arena_len = before;
        return S2P_OK;
    }
    /* the quantiser that produced the tensors ran on `stream`: both downloads follow it there */
    S2P_CUDA_TRY(cudaMemcpyAsync(qc->arena + e.q_off, codes->data, codes->bytes, cudaMemcpyDeviceToHost, stream));
    S2P_CUDA_TRY(cudaMemcpyAsync(qc->arena + e.s_off, lin->w_iscale.data, lin->w_iscale.bytes, cudaMemcpyDeviceToHost, stream));
    S2P_CUDA_TRY(cudaStreamSynchronize(stream)); /* pageable destination that may move when the arena grows */
    qc->entries[qc->n++] = e;
    return S2P_OK;
}

static int write_at(int fd, const void* data, size_t len, uint64_t off) {
    const unsigned char* p = (const unsigned char*)data;
    while (len) {
        const ssize_t w = pwrite(fd, p, len, (off_t)off);
        if (w < 0 && errno == EINTR) continue;
        if (w <= 0) return 0;
        p += w; off += (uint64_t)w; len -= (size_t)w;
    }
    return 1;
}
static uint64_t align_up(uint64_t v) { return (v + (QC_ALIGN - 1)) & ~(uint64_t)(QC_ALIGN - 1); }

s2p_status s2p_qcache_finish(s2p_qcache* qc, cudaStream_t stream) {
    if (!qc) return S2P_OK;
    if (qc->reading) { /* the queued uploads read from the mapping: they must have landed before it goes */
        S2P_CUDA_TRY(cudaStreamSynchronize(stream));
        unmap_file(qc);
        return S2P_OK;
    }
    if (!qc->n) return S2P_OK;
    /* layout: header, entry table, then every region at the next 256-byte boundary */
    uint64_t table = QC_HEADER_BYTES;
    for (int i = 0; i < qc->n; i++) table += QC_ENTRY_BYTES + strlen(qc->entries[i].name);
    unsigned char* head = (unsigned char*)calloc(1, (size_t)table);
    uint64_t* file_q = (uint64_t*)malloc((size_t)qc->n * 2 * sizeof(uint64_t));
    if (!head || !file_q) { free(head); free(file_q); return S2P_OK; }
    uint64_t end = table;
    for (int i = 0; i < qc->n; i++) {
        file_q[2 * i] = end = align_up(end); end += qc->entries[i].q_len;
        file_q[2 * i + 1] = end = align_up(end); end += qc->entries[i].s_len;
    }
    memcpy(head, QC_MAGIC, 8);
    memcpy(head + 8, &qc->fingerprint, 8);
    const uint32_t n32 = (uint32_t)qc->n;
    memcpy(head + 16, &n32, 4);
    uint64_t at = QC_HEADER_BYTES;
    for (int i = 0; i < qc->n; i++) {
        const qc_entry* e = &qc->entries[i];
        const uint32_t name_len = (uint32_t)strlen(e->name);
        unsigned char* rec = head + at;
        memcpy(rec, &name_len, 4); memcpy(rec + 4, &e->kind, 4); memcpy(rec + 8, &e->N, 4);
        memcpy(rec + 12, &e->K, 4); memcpy(rec + 16, &e->group, 4);
        memcpy(rec + 24, &file_q[2 * i], 8); memcpy(rec + 32, &e->q_len, 8);
        memcpy(rec + 40, &file_q[2 * i + 1], 8); memcpy(rec + 48, &e->s_len, 8);
        memcpy(rec + QC_ENTRY_BYTES, e->name, name_len);
        at += QC_ENTRY_BYTES + name_len;
    }
    char tmp[1200];
    snprintf(tmp, sizeof(tmp), "%s.tmp", qc->path);
    const int fd = open(tmp, O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) {
        fprintf(stderr, "[s2pro] qcache: cannot write %s (skipping)\n", tmp);
        free(head); free(file_q);
        return S2P_OK;
    }
    int ok = ftruncate(fd, (off_t)end) == 0 && write_at(fd, head, (size_t)table, 0); /* the gaps read as zeros */
    for (int i = 0; ok && i < qc->n; i++) {
        const qc_entry* e = &qc->entries[i];
        ok = write_at(fd, qc->arena + e->q_off, e->q_len, file_q[2 * i]) && write_at(fd, qc->arena + e->s_off, e->s_len, file_q[2 * i + 1]);
    }
    ok = (close(fd) == 0) && ok;
    free(head);
    free(file_q);
    if (!ok || rename(tmp, qc->path) != 0) {
        fprintf(stderr, "[s2pro] qcache: write failed (%s), removing\n", tmp);
        unlink(tmp);
        return S2P_OK;
    }
    fprintf(stderr, "[s2pro] qcache: wrote %d tensors -> %s\n", qc->n, qc->path);
    return S2P_OK;
}

void s2p_qcache_free(s2p_qcache* qc) {
    if (!qc) return;
    drop_entries(qc);
    unmap_file(qc);
    free(qc->arena);
    free(qc);
}
