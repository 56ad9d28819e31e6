/* Checkpoint reader for the weight-loader contract
 * (include/s2pro/safetensors.h:17-38 of the reference; behaviour follows
 * src/core/safetensors.c:133-509: one model.safetensors or the shards named by
 * model.safetensors.index.json, files mapped read-only until close, duplicate
 * names rejected).
 *
 * A safetensors file is: u64 little-endian header length, a JSON object whose
 * members map tensor names to {"dtype","shape","data_offsets"}, then the data
 * section the offsets are relative to.  The header grammar is small and flat,
 * so it is scanned directly here instead of going through a general JSON tree.
 */
#include <fcntl.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include "s2p_b200_abi.h"

typedef struct { char* name; s2p_st_view v; } entry;
typedef struct { unsigned char* map; size_t size; } mapped;

struct s2p_st {
    mapped* files; int nfiles;
    entry* ents; int count, cap;
    int* slots; unsigned mask; /* open-addressing index: entry+1, 0 = empty */
};

/* ---- tiny JSON cursor ---- */
typedef struct { const char* p; const char* end; } cur;

static void ws(cur* c) { while (c->p < c->end && (*c->p == ' ' || *c->p == '\n' || *c->p == '\t' || *c->p == '\r')) c->p++; }
static int eat(cur* c, char ch) { ws(c); if (c->p < c->end && *c->p == ch) { c->p++; return 1; } return 0; }

/* Parse a JSON string into a fresh NUL-terminated buffer (escapes \" \\ \/ \n \t \uXXXX-as-is). */
static char* jstring(cur* c) {
    ws(c);
    if (c->p >= c->end || *c->p != '"') return NULL;
    const char* s = ++c->p;
    size_t cap = 64, n = 0;
    char* out = (char*)malloc(cap);
    if (!out) return NULL;
    while (s < c->end && *s != '"') {
        char ch = *s++;
        if (ch == '\\' && s < c->end) {
            char e = *s++;
            ch = e == 'n' ? '\n' : e == 't' ? '\t' : e == 'r' ? '\r' : e == 'b' ? '\b' : e == 'f' ? '\f' : e;
        }
        if (n + 2 > cap) { cap *= 2; char* t = (char*)realloc(out, cap); if (!t) { free(out); return NULL; } out = t; }
        out[n++] = ch;
    }
    if (s >= c->end) { free(out); return NULL; }
    out[n] = 0;
    c->p = s + 1;
    return out;
}

static int jint(cur* c, int64_t* out) {
    ws(c);
    if (c->p >= c->end || (*c->p < '0' || *c->p > '9')) return 0;
    int64_t v = 0;
    while (c->p < c->end && *c->p >= '0' && *c->p <= '9') {
        if (v > (INT64_MAX - 9) / 10) return 0;
        v = v * 10 + (*c->p++ - '0');
    }
    *out = v;
    return 1;
}

/* Skip any JSON value (used for __metadata__ and unknown members). */
static int jskip(cur* c) {
    ws(c);
    if (c->p >= c->end) return 0;
    const char ch = *c->p;
    if (ch == '"') { char* s = jstring(c); if (!s) return 0; free(s); return 1; }
    if (ch == '{' || ch == '[') {
        const char close = ch == '{' ? '}' : ']';
        c->p++;
        if (eat(c, close)) return 1;
        for (;;) {
            if (ch == '{') { char* k = jstring(c); if (!k) return 0; free(k); if (!eat(c, ':')) return 0; }
            if (!jskip(c)) return 0;
            if (eat(c, ',')) continue;
            return eat(c, close);
        }
    }
    while (c->p < c->end && *c->p != ',' && *c->p != '}' && *c->p != ']') c->p++;
    return 1;
}

static int dtype_of(const char* s, s2p_dtype* dt) {
    static const struct { const char* n; s2p_dtype d; } tab[] = {
        {"BF16", S2P_DT_BF16}, {"F16", S2P_DT_F16}, {"F32", S2P_DT_F32}, {"I64", S2P_DT_I64},
        {"I32", S2P_DT_I32}, {"U8", S2P_DT_U8}, {"I8", S2P_DT_I8}, {"BOOL", S2P_DT_U8}};
    for (size_t i = 0; i < sizeof(tab) / sizeof(tab[0]); i++)
        if (!strcmp(s, tab[i].n)) { *dt = tab[i].d; return 1; }
    return 0;
}

static s2p_status push(s2p_st* st, char* name, const s2p_st_view* v) {
    if (st->count == st->cap) {
        const int nc = st->cap ? st->cap * 2 : 512;
        entry* ne = (entry*)realloc(st->ents, (size_t)nc * sizeof(entry));
        if (!ne) return S2P_ERR_OOM;
        st->ents = ne; st->cap = nc;
    }
    st->ents[st->count].name = name;
    st->ents[st->count].v = *v;
    st->ents[st->count].v.name = name;
    st->count++;
    return S2P_OK;
}

static s2p_status map_file(s2p_st* st, const char* dir, const char* fname) {
    char path[2048];
    if (snprintf(path, sizeof(path), "%s/%s", dir, fname) >= (int)sizeof(path)) return S2P_ERR_INVALID;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return S2P_ERR_IO;
    struct stat sb;
    if (fstat(fd, &sb) != 0 || sb.st_size < 8) { close(fd); return sb.st_size < 8 ? S2P_ERR_FORMAT : S2P_ERR_IO; }
    unsigned char* map = (unsigned char*)mmap(NULL, (size_t)sb.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) return S2P_ERR_IO;
    mapped* nf = (mapped*)realloc(st->files, (size_t)(st->nfiles + 1) * sizeof(mapped));
    if (!nf) { munmap(map, (size_t)sb.st_size); return S2P_ERR_OOM; }
    st->files = nf;
    st->files[st->nfiles].map = map;
    st->files[st->nfiles].size = (size_t)sb.st_size;
    st->nfiles++;

    uint64_t hlen = 0;
    for (int i = 7; i >= 0; i--) hlen = (hlen << 8) | map[i];
    if (hlen > (uint64_t)sb.st_size - 8) return S2P_ERR_FORMAT;
    const unsigned char* data = map + 8 + hlen;
    const size_t data_len = (size_t)sb.st_size - 8 - (size_t)hlen;
    cur c = {(const char*)map + 8, (const char*)map + 8 + hlen};
    if (!eat(&c, '{')) return S2P_ERR_FORMAT;
    if (eat(&c, '}')) return S2P_OK;
    for (;;) {
        char* name = jstring(&c);
        if (!name || !eat(&c, ':')) { free(name); return S2P_ERR_FORMAT; }
        if (!strcmp(name, "__metadata__")) {
            free(name);
            if (!jskip(&c)) return S2P_ERR_FORMAT;
        } else {
            s2p_st_view v;
            memset(&v, 0, sizeof(v));
            int have_dt = 0, have_shape = 0, have_off = 0;
            int64_t b0 = 0, b1 = 0;
            if (!eat(&c, '{')) { free(name); return S2P_ERR_FORMAT; }
            for (;;) {
                char* key = jstring(&c);
                if (!key || !eat(&c, ':')) { free(key); free(name); return S2P_ERR_FORMAT; }
                int ok = 1;
                if (!strcmp(key, "dtype")) {
                    char* d = jstring(&c);
                    ok = d != NULL;
                    if (d && !dtype_of(d, &v.dtype)) { free(d); free(key); free(name); return S2P_ERR_UNSUPPORTED; }
                    free(d);
                    have_dt = 1;
                } else if (!strcmp(key, "shape")) {
                    ok = eat(&c, '[');
                    v.ndim = 0;
                    if (ok && !eat(&c, ']')) {
                        do {
                            int64_t d;
                            if (v.ndim >= 4 || !jint(&c, &d)) { ok = 0; break; }
                            v.shape[v.ndim++] = d;
                        } while (eat(&c, ','));
                        ok = ok && eat(&c, ']');
                    }
                    have_shape = 1;
                } else if (!strcmp(key, "data_offsets")) {
                    ok = eat(&c, '[') && jint(&c, &b0) && eat(&c, ',') && jint(&c, &b1) && eat(&c, ']');
                    have_off = 1;
                } else {
                    ok = jskip(&c);
                }
                free(key);
                if (!ok) { free(name); return S2P_ERR_FORMAT; }
                if (eat(&c, ',')) continue;
                if (!eat(&c, '}')) { free(name); return S2P_ERR_FORMAT; }
                break;
            }
            if (!have_dt || !have_shape || !have_off || b1 < b0 || (uint64_t)b1 > data_len) {
                free(name);
                return S2P_ERR_FORMAT;
            }
            int64_t numel = 1;
            for (int i = 0; i < v.ndim; i++) numel *= v.shape[i];
            for (int i = v.ndim; i < 4; i++) v.shape[i] = 1;
            if ((uint64_t)numel * s2p_dtype_size(v.dtype) != (uint64_t)(b1 - b0)) { free(name); return S2P_ERR_FORMAT; }
            v.data = data + b0;
            v.nbytes = (size_t)(b1 - b0);
            const s2p_status rc = push(st, name, &v);
            if (rc != S2P_OK) { free(name); return rc; }
        }
        if (eat(&c, ',')) continue;
        return eat(&c, '}') ? S2P_OK : S2P_ERR_FORMAT;
    }
}

static uint64_t hash_name(const char* s) {
    uint64_t h = 1469598103934665603ull;
    while (*s) { h ^= (unsigned char)*s++; h *= 1099511628211ull; }
    return h;
}

static s2p_status build_index(s2p_st* st) {
    unsigned n = 16;
    while (n < (unsigned)st->count * 2u + 1u) n <<= 1;
    st->slots = (int*)calloc(n, sizeof(int));
    if (!st->slots) return S2P_ERR_OOM;
    st->mask = n - 1;
    for (int i = 0; i < st->count; i++) {
        unsigned h = (unsigned)hash_name(st->ents[i].name) & st->mask;
        while (st->slots[h]) {
            if (!strcmp(st->ents[st->slots[h] - 1].name, st->ents[i].name)) return S2P_ERR_FORMAT; /* duplicate */
            h = (h + 1) & st->mask;
        }
        st->slots[h] = i + 1;
    }
    return S2P_OK;
}

/* The index file maps tensor names to shard file names under "weight_map";
 * only the distinct shard names matter (every tensor of every shard is indexed). */
static s2p_status open_sharded(s2p_st* st, const char* dir, const char* index_path) {
    FILE* f = fopen(index_path, "rb");
    if (!f) return S2P_ERR_IO;
    fseek(f, 0, SEEK_END);
    const long sz = ftell(f);
    fseek(f, 0, SEEK_SET);
    char* buf = sz > 0 ? (char*)malloc((size_t)sz) : NULL;
    if (!buf || fread(buf, 1, (size_t)sz, f) != (size_t)sz) { free(buf); fclose(f); return buf ? S2P_ERR_IO : S2P_ERR_OOM; }
    fclose(f);
    cur c = {buf, buf + sz};
    s2p_status rc = S2P_ERR_FORMAT;
    char* seen[256];
    int nseen = 0;
    if (!eat(&c, '{')) goto done;
    for (;;) {
        char* key = jstring(&c);
        if (!key || !eat(&c, ':')) { free(key); goto done; }
        if (!strcmp(key, "weight_map")) {
            free(key);
            if (!eat(&c, '{')) goto done;
            if (!eat(&c, '}')) for (;;) {
                char* tn = jstring(&c);
                if (!tn || !eat(&c, ':')) { free(tn); goto done; }
                free(tn);
                char* shard = jstring(&c);
                if (!shard) goto done;
                int dup = 0;
                for (int i = 0; i < nseen; i++) if (!strcmp(seen[i], shard)) dup = 1;
                if (dup || nseen == 256) free(shard); else seen[nseen++] = shard;
                if (eat(&c, ',')) continue;
                if (!eat(&c, '}')) goto done;
                break;
            }
        } else {
            free(key);
            if (!jskip(&c)) goto done;
        }
        if (eat(&c, ',')) continue;
        if (!eat(&c, '}')) goto done;
        break;
    }
    rc = nseen ? S2P_OK : S2P_ERR_FORMAT;
    for (int i = 0; i < nseen && rc == S2P_OK; i++) rc = map_file(st, dir, seen[i]);
done:
    for (int i = 0; i < nseen; i++) free(seen[i]);
    free(buf);
    return rc;
}

s2p_status s2p_st_open_dir(const char* model_dir, s2p_st** out) {
    if (!model_dir || !out) return S2P_ERR_INVALID;
    *out = NULL;
    s2p_st* st = (s2p_st*)calloc(1, sizeof(*st));
    if (!st) return S2P_ERR_OOM;
    char path[2048];
    snprintf(path, sizeof(path), "%s/model.safetensors.index.json", model_dir);
    s2p_status rc = access(path, R_OK) == 0 ? open_sharded(st, model_dir, path)
                                             : map_file(st, model_dir, "model.safetensors");
    if (rc == S2P_OK) rc = build_index(st);
    if (rc != S2P_OK) { s2p_st_close(st); return rc; }
    *out = st;
    return S2P_OK;
}

s2p_status s2p_st_find(s2p_st* st, const char* name, s2p_st_view* out) {
    if (!st || !name || !out || !st->slots) return S2P_ERR_INVALID;
    unsigned h = (unsigned)hash_name(name) & st->mask;
    while (st->slots[h]) {
        const entry* e = &st->ents[st->slots[h] - 1];
        if (!strcmp(e->name, name)) { *out = e->v; return S2P_OK; }
        h = (h + 1) & st->mask;
    }
    return S2P_ERR_INVALID;
}

int s2p_st_count(const s2p_st* st) { return st ? st->count : 0; }

s2p_status s2p_st_at(const s2p_st* st, int index, s2p_st_view* out) {
    if (!st || !out || index < 0 || index >= st->count) return S2P_ERR_INVALID;
    *out = st->ents[index].v;
    return S2P_OK;
}

void s2p_st_close(s2p_st* st) {
    if (!st) return;
    for (int i = 0; i < st->count; i++) free(st->ents[i].name);
    for (int i = 0; i < st->nfiles; i++) munmap(st->files[i].map, st->files[i].size);
    free(st->ents); free(st->files); free(st->slots); free(st);
}

s2p_status s2p_st_load_device(s2p_st* st, const char* name, s2p_dtype expect_dt, int ndim,
                              const int64_t* expect_shape, s2p_tensor* out_dev, cudaStream_t stream) {
    if (!out_dev) return S2P_ERR_INVALID;
    s2p_st_view v;
    if (s2p_st_find(st, name, &v) != S2P_OK) {
        fprintf(stderr, "[s2pro] checkpoint tensor missing: %s\n", name ? name : "(null)");
        return S2P_ERR_INVALID; /* same status as a failed s2p_st_find */
    }
    if (v.dtype != expect_dt || v.ndim != ndim) return S2P_ERR_FORMAT;
    for (int i = 0; i < ndim; i++)
        if (expect_shape && expect_shape[i] >= 0 && expect_shape[i] != v.shape[i]) return S2P_ERR_FORMAT;
    S2P_TRY(s2p_tensor_device_alloc(out_dev, v.dtype, v.ndim, v.shape));
    const s2p_status rc = s2p_tensor_upload(out_dev, v.data, v.nbytes, stream);
    if (rc != S2P_OK) s2p_tensor_free(out_dev);
    return rc;
}
