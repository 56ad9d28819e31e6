/* Prequantised-weight sidecar (reference contract include/s2pro/qcache.h:34-54;
 * file format and staleness rule of src/sched/qcache.c:3-17, 74-113).
 *
 * Quantising a checkpoint at load (per-channel INT8, group-wise INT4 with the
 * clip search) is repeated work on every start; the sidecar stores the final
 * device tensors once and later starts upload them as they are.  The file is
 * interchangeable with the reference's:
 *
 *   "S2PQC\1\0\0" | u64 fingerprint | u32 n | u32 0
 *   n x { u32 name_len, u32 kind, i32 N, i32 K, i32 group, u32 0,
 *         u64 q_off, u64 q_len, u64 s_off, u64 s_len, name bytes }
 *   payloads at 256-byte aligned absolute offsets
 *   kind 1: i8[N,K] + f32[N]; 2: nibbles[N,K/2] + f16[N*K/G]; 3: i8[N,K] + f16[N*K/G]
 *
 * The fingerprint is FNV-1a over the quantisation settings and the (name, size,
 * mtime) of every *.safetensors in the model directory; a mismatch or any read
 * problem means "miss" and the live quantisers run.  S2P_QCACHE=0 disables the
 * sidecar, S2P_QCACHE_DIR moves it.
 */
#include <dirent.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include "internal.h"

#define QC_MAX 512
#define QC_HDR 24
#define QC_ENT 56

typedef struct {
    char* name;
    uint32_t kind;
    int32_t N, K, group;
    uint64_t q_off, q_len, s_off, s_len;
    void *q_host, *s_host; /* write mode */
} qent;

struct s2p_qcache {
    char path[1100];
    int reading;
    uint64_t fingerprint;
    unsigned char* file; /* read mode: the whole sidecar */
    size_t file_len;
    qent e[QC_MAX];
    int n;
};

static uint64_t fnv(uint64_t h, const void* data, size_t len) {
    const unsigned char* p = (const unsigned char*)data;
    while (len--) { h ^= *p++; h *= 0x100000001b3ULL; }
    return h;
}
static int flag(const char* name, int def) {
    const char* v = getenv(name);
    return (v && v[0]) ? (v[0] == '1' && v[1] == '\0') : def;
}
static int by_name(const void* a, const void* b) { return strcmp(*(char* const*)a, *(char* const*)b); }

static int fingerprint(const char* dir, s2p_gemm_mode mode, uint64_t* out) {
    char cfg[256];
    const char* g = getenv("S2P_INT4_GROUP");
    snprintf(cfg, sizeof(cfg), "v1|mode=%d|int4=%d|g=%s|mse=%d|pk=%d|all=%d", (int)mode, flag("S2P_INT4", 0),
             g ? g : "32", flag("S2P_INT4_MSE", 1), flag("S2P_INT4_PACKED", 1), flag("S2P_INT4_ALL", 0));
    uint64_t h = fnv(0xcbf29ce484222325ULL, cfg, strlen(cfg));
    DIR* d = opendir(dir);
    if (!d) return 0;
    char* names[256];
    int n = 0;
    for (struct dirent* de; (de = readdir(d)) != NULL && n < 256;) {
        const size_t len = strlen(de->d_name);
        if (len > 12 && !strcmp(de->d_name + len - 12, ".safetensors")) names[n++] = strdup(de->d_name);
    }
    closedir(d);
    if (!n) return 0;
    qsort(names, (size_t)n, sizeof(names[0]), by_name);
    for (int i = 0; i < n; i++) {
        char full[1400];
        struct stat sb;
        snprintf(full, sizeof(full), "%s/%s", dir, names[i]);
        if (stat(full, &sb) == 0) {
            h = fnv(h, names[i], strlen(names[i]));
            h = fnv(h, &sb.st_size, sizeof(sb.st_size));
            h = fnv(h, &sb.st_mtime, sizeof(sb.st_mtime));
        }
        free(names[i]);
    }
    *out = h;
    return 1;
}

static uint64_t rd64(const unsigned char* p) { uint64_t v; memcpy(&v, p, 8); return v; }
static uint32_t rd32(const unsigned char* p) { uint32_t v; memcpy(&v, p, 4); return v; }

/* Parse an existing sidecar; leaves the handle in write mode on any inconsistency. */
static void try_read(s2p_qcache* qc) {
    FILE* f = fopen(qc->path, "rb");
    if (!f) return;
    fseek(f, 0, SEEK_END);
    const long sz = ftell(f);
    fseek(f, 0, SEEK_SET);
    unsigned char* buf = sz >= QC_HDR ? (unsigned char*)malloc((size_t)sz) : NULL;
    const int ok = buf && fread(buf, 1, (size_t)sz, f) == (size_t)sz;
    fclose(f);
    if (!ok || memcmp(buf, "S2PQC\1\0\0", 8) != 0) { free(buf); return; }
    if (rd64(buf + 8) != qc->fingerprint) {
        fprintf(stderr, "[s2pro] qcache: stale fingerprint, rebuilding\n");
        free(buf);
        return;
    }
    const uint32_t n = rd32(buf + 16);
    if (n == 0 || n > QC_MAX) { free(buf); return; }
    size_t off = QC_HDR;
    uint32_t i = 0;
    for (; i < n; i++) {
        if (off + QC_ENT > (size_t)sz) break;
        qent* e = &qc->e[i];
        const uint32_t name_len = rd32(buf + off);
        e->kind = rd32(buf + off + 4);
        e->N = (int32_t)rd32(buf + off + 8);
        e->K = (int32_t)rd32(buf + off + 12);
        e->group = (int32_t)rd32(buf + off + 16);
        e->q_off = rd64(buf + off + 24);
        e->q_len = rd64(buf + off + 32);
        e->s_off = rd64(buf + off + 40);
        e->s_len = rd64(buf + off + 48);
        off += QC_ENT;
        if (!name_len || name_len > 512 || off + name_len > (size_t)sz) break;
        if (e->q_off + e->q_len > (uint64_t)sz || e->s_off + e->s_len > (uint64_t)sz) break;
        e->name = (char*)malloc(name_len + 1);
        if (!e->name) break;
        memcpy(e->name, buf + off, name_len);
        e->name[name_len] = 0;
        off += name_len;
    }
    if (i != n) {
        for (uint32_t j = 0; j <= i && j < n; j++) { free(qc->e[j].name); qc->e[j].name = NULL; }
        free(buf);
        return;
    }
    qc->file = buf;
    qc->file_len = (size_t)sz;
    qc->n = (int)n;
    qc->reading = 1;
}

s2p_status s2p_qcache_open(const char* model_dir, s2p_gemm_mode mode, s2p_qcache** out) {
    if (!model_dir || !out) return S2P_ERR_INVALID;
    *out = NULL;
    if (mode != S2P_GEMM_INT8 || !flag("S2P_QCACHE", 1)) return S2P_OK;
    s2p_qcache* qc = (s2p_qcache*)calloc(1, sizeof(*qc));
    if (!qc) return S2P_ERR_OOM;
    if (!fingerprint(model_dir, mode, &qc->fingerprint)) { free(qc); return S2P_OK; }
    const char* dir = getenv("S2P_QCACHE_DIR");
    snprintf(qc->path, sizeof(qc->path), "%s/s2p_qcache.bin", (dir && dir[0]) ? dir : model_dir);
    try_read(qc);
    if (qc->reading) fprintf(stderr, "[s2pro] qcache: serving %d tensors from %s\n", qc->n, qc->path);
    else fprintf(stderr, "[s2pro] qcache: will write %s after load\n", qc->path);
    *out = qc;
    return S2P_OK;
}

int s2p_qcache_reading(const s2p_qcache* qc) { return qc && qc->reading; }

int s2p_qcache_try_load(s2p_qcache* qc, const char* name, int in_features, int out_features, s2p_linear* lin,
                        cudaStream_t stream) {
    if (!qc || !qc->reading || !name || !lin) return 0;
    const qent* e = NULL;
    for (int i = 0; i < qc->n && !e; i++)
        if (!strcmp(qc->e[i].name, name)) e = &qc->e[i];
    if (!e) { fprintf(stderr, "[s2pro] qcache: miss for %s (live path)\n", name); return 0; }
    if (e->N != out_features || e->K != in_features || e->kind < 1 || e->kind > 3 ||
        (e->kind >= 2 && (e->group <= 0 || e->K % e->group))) {
        fprintf(stderr, "[s2pro] qcache: shape mismatch for %s\n", name);
        return 0;
    }
    memset(lin, 0, sizeof(*lin));
    lin->in_features = in_features;
    lin->out_features = out_features;
    s2p_tensor* qt = e->kind == 2 ? &lin->w_pack : &lin->w_int8;
    const int64_t qshape[2] = {e->N, e->kind == 2 ? e->K / 2 : e->K};
    const int64_t sshape[1] = {e->kind == 1 ? e->N : (int64_t)e->N * (e->K / e->group)};
    s2p_status rc = s2p_tensor_device_alloc(qt, S2P_DT_I8, 2, qshape);
    if (rc == S2P_OK) rc = s2p_tensor_device_alloc(&lin->w_iscale, e->kind == 1 ? S2P_DT_F32 : S2P_DT_F16, 1, sshape);
    if (rc == S2P_OK && (qt->bytes != e->q_len || lin->w_iscale.bytes != e->s_len)) rc = S2P_ERR_FORMAT;
    if (rc == S2P_OK) rc = s2p_tensor_upload(qt, qc->file + e->q_off, e->q_len, stream);
    if (rc == S2P_OK) rc = s2p_tensor_upload(&lin->w_iscale, qc->file + e->s_off, e->s_len, stream);
    if (rc != S2P_OK) {
        s2p_tensor_free(qt);
        s2p_tensor_free(&lin->w_iscale);
        memset(lin, 0, sizeof(*lin));
        lin->in_features = in_features;
        lin->out_features = out_features;
        return 0;
    }
    lin->int8_ready = 1;
    if (e->kind >= 2) lin->q_group = e->group;
    if (e->kind == 2) lin->q_packed = 1;
    return 1;
}

s2p_status s2p_qcache_put_linear(s2p_qcache* qc, const char* name, const s2p_linear* lin, cudaStream_t stream) {
    if (!qc || qc->reading || !name || !lin || !lin->int8_ready || qc->n >= QC_MAX) return S2P_OK;
    const s2p_tensor* qt = lin->q_packed ? &lin->w_pack : &lin->w_int8;
    if (!qt->data || !lin->w_iscale.data) return S2P_OK;
    qent* e = &qc->e[qc->n];
    memset(e, 0, sizeof(*e));
    e->kind = lin->q_packed ? 2u : (lin->q_group > 0 ? 3u : 1u);
    e->N = lin->out_features;
    e->K = lin->in_features;
    e->group = lin->q_group;
    e->q_len = qt->bytes;
    e->s_len = lin->w_iscale.bytes;
    e->q_host = malloc(qt->bytes);
    e->s_host = malloc(lin->w_iscale.bytes);
    e->name = strdup(name);
    if (!e->q_host || !e->s_host || !e->name) { /* the cache degrades, the load does not */
        free(e->q_host); free(e->s_host); free(e->name);
        memset(e, 0, sizeof(*e));
        return S2P_OK;
    }
    S2P_CUDA_TRY(cudaStreamSynchronize(stream));
    S2P_CUDA_TRY(cudaMemcpy(e->q_host, qt->data, qt->bytes, cudaMemcpyDeviceToHost));
    S2P_CUDA_TRY(cudaMemcpy(e->s_host, lin->w_iscale.data, lin->w_iscale.bytes, cudaMemcpyDeviceToHost));
    qc->n++;
    return S2P_OK;
}

static int pad_to(FILE* f, uint64_t target) {
    static const char zeros[256] = {0};
    long pos = ftell(f);
    while (pos >= 0 && (uint64_t)pos < target) {
        size_t n = (size_t)(target - (uint64_t)pos);
        if (n > sizeof(zeros)) n = sizeof(zeros);
        if (fwrite(zeros, 1, n, f) != n) return 0;
        pos = ftell(f);
    }
    return pos >= 0;
}

s2p_status s2p_qcache_finish(s2p_qcache* qc, cudaStream_t stream) {
    if (!qc) return S2P_OK;
    if (qc->reading) { /* uploads read from the file buffer: they must have landed */
        S2P_CUDA_TRY(cudaStreamSynchronize(stream));
        free(qc->file);
        qc->file = NULL;
        return S2P_OK;
    }
    if (!qc->n) return S2P_OK;
    uint64_t off = QC_HDR;
    for (int i = 0; i < qc->n; i++) off += QC_ENT + strlen(qc->e[i].name);
    for (int i = 0; i < qc->n; i++) {
        qent* e = &qc->e[i];
        off = (off + 255) & ~255ull; e->q_off = off; off += e->q_len;
        off = (off + 255) & ~255ull; e->s_off = off; off += e->s_len;
    }
    char tmp[1200];
    snprintf(tmp, sizeof(tmp), "%s.tmp", qc->path);
    FILE* f = fopen(tmp, "wb");
    if (!f) { fprintf(stderr, "[s2pro] qcache: cannot write %s (skipping)\n", tmp); return S2P_OK; }
    const uint32_t n32 = (uint32_t)qc->n, zero = 0;
    int ok = fwrite("S2PQC\1\0\0", 1, 8, f) == 8 && fwrite(&qc->fingerprint, 8, 1, f) == 1 &&
             fwrite(&n32, 4, 1, f) == 1 && fwrite(&zero, 4, 1, f) == 1;
    for (int i = 0; i < qc->n && ok; i++) {
        const qent* e = &qc->e[i];
        const uint32_t nl = (uint32_t)strlen(e->name);
        ok = fwrite(&nl, 4, 1, f) == 1 && fwrite(&e->kind, 4, 1, f) == 1 && fwrite(&e->N, 4, 1, f) == 1 &&
             fwrite(&e->K, 4, 1, f) == 1 && fwrite(&e->group, 4, 1, f) == 1 && fwrite(&zero, 4, 1, f) == 1 &&
             fwrite(&e->q_off, 8, 1, f) == 1 && fwrite(&e->q_len, 8, 1, f) == 1 && fwrite(&e->s_off, 8, 1, f) == 1 &&
             fwrite(&e->s_len, 8, 1, f) == 1 && fwrite(e->name, 1, nl, f) == nl;
    }
    for (int i = 0; i < qc->n && ok; i++) {
        const qent* e = &qc->e[i];
        ok = pad_to(f, e->q_off) && fwrite(e->q_host, 1, e->q_len, f) == e->q_len && pad_to(f, e->s_off) &&
             fwrite(e->s_host, 1, e->s_len, f) == e->s_len;
    }
    ok = (fclose(f) == 0) && ok;
    if (!ok || rename(tmp, qc->path) != 0) {
        fprintf(stderr, "[s2pro] qcache: write failed (%s), removing\n", tmp);
        remove(tmp);
        return S2P_OK;
    }
    fprintf(stderr, "[s2pro] qcache: wrote %d tensors -> %s\n", qc->n, qc->path);
    return S2P_OK;
}

void s2p_qcache_free(s2p_qcache* qc) {
    if (!qc) return;
    for (int i = 0; i < qc->n; i++) { free(qc->e[i].name); free(qc->e[i].q_host); free(qc->e[i].s_host); }
    free(qc->file);
    free(qc);
}
