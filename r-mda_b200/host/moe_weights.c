/*
 * moe_weights.c -- safetensors shards -> staging banks -> device fp16 (see
 * moe_weights.h for the reference functions each part stands in for).
 *
 * A safetensors file is: 8 bytes little-endian header length, a JSON object
 * { "<tensor name>": {"dtype": "...", "shape": [...], "data_offsets": [a, b]}, ...,
 *   "__metadata__": {...} }, then the tensor bytes; offsets count from the end
 * of the header.  The header is scanned once into a table when the file is
 * mapped; nothing is copied until a tensor is staged.
 */
#define _GNU_SOURCE
#include "moe_weights.h"

#include <dirent.h>
#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

/* ---- a scanner for the subset of JSON a safetensors header uses -------------- */

typedef struct moe_json_t {
    const char *p, *end;
    bool bad;
} moe_json_t;

static void js_space(moe_json_t *j) {
    while (j->p < j->end && (*j->p == ' ' || *j->p == '\n' || *j->p == '\t' || *j->p == '\r')) {
        j->p += 1;
    }
}

static bool js_take(moe_json_t *j, char ch) {
    js_space(j);
    if (j->p < j->end && *j->p == ch) {
        j->p += 1;
        return true;
    }
    return false;
}

/* A string token; the span excludes the quotes and keeps escapes as written. */
static bool js_string(moe_json_t *j, const char **s, uint32_t *n) {
    if (js_take(j, '"') == false) {
        j->bad = true;
        return false;
    }
    const char *start = j->p;
    while (j->p < j->end && *j->p != '"') {
        j->p += (*j->p == '\\') ? 2 : 1;
    }
    if (j->p >= j->end) {
        j->bad = true;
        return false;
    }
    *s = start;
    *n = (uint32_t)(j->p - start);
    j->p += 1;
    return true;
}

static uint64_t js_number(moe_json_t *j) {
    js_space(j);
    uint64_t v = 0;
    bool any = false;
    while (j->p < j->end && *j->p >= '0' && *j->p <= '9') {
        v = v * 10 + (uint64_t)(*j->p - '0');
        j->p += 1;
        any = true;
    }
    if (any == false) {
        j->bad = true;
    }
    return v;
}

static void js_skip(moe_json_t *j) { /* any value */
    js_space(j);
    if (j->p >= j->end) {
        j->bad = true;
    } else if (*j->p == '"') {
        const char *s;
        uint32_t n;
        js_string(j, &s, &n);
    } else if (*j->p == '{' || *j->p == '[') {
        uint32_t depth = 0;
        while (j->p < j->end && j->bad == false) {
            char ch = *j->p;
            if (ch == '"') {
                const char *s;
                uint32_t n;
                js_string(j, &s, &n);
                continue;
            }
            j->p += 1;
            if (ch == '{' || ch == '[') {
                depth += 1;
            } else if (ch == '}' || ch == ']') {
                depth -= 1;
                if (depth == 0) {
                    return;
                }
            }
        }
        j->bad = true;
    } else {
        while (j->p < j->end && *j->p != ',' && *j->p != '}' && *j->p != ']') {
            j->p += 1;
        }
    }
}

static bool span_is(const char *s, uint32_t n, const char *lit) {
    return strlen(lit) == n && memcmp(s, lit, n) == 0;
}

static void st_dtype(moe_st_entry_t *e, const char *s, uint32_t n) {
    static const struct {
        const char *name;
        uint32_t elem;
    } known[] = {{"F64", 8}, {"F32", 4}, {"F16", 2}, {"I32", 4}, {"I16", 2}, {"I8", 1},      {"U8", 1},
                 {"U16", 2}, {"U32", 4}, {"U64", 8}, {"BOOL", 1}, {"F8_E4M3", 1}, {"F8_E5M2", 1}};
    e->dtype = MOE_ST_OTHER;
    e->elem = 0;
    if (span_is(s, n, "BF16")) {
        e->dtype = MOE_ST_BF16;
        e->elem = 2;
    } else if (span_is(s, n, "I64")) {
        e->dtype = MOE_ST_I64;
        e->elem = 8;
    } else {
        for (uint32_t i = 0; i < sizeof(known) / sizeof(known[0]); i += 1) {
            if (span_is(s, n, known[i].name)) {
                e->elem = known[i].elem;
            }
        }
    }
}

static void st_entry(moe_json_t *j, moe_st_entry_t *e) { /* {"dtype":..,"shape":[..],"data_offsets":[a,b]} */
    if (js_take(j, '{') == false) {
        j->bad = true;
        return;
    }
    bool have_dtype = false, have_shape = false, have_offs = false;
    while (j->bad == false && js_take(j, '}') == false) {
        const char *k;
        uint32_t kn;
        if (js_string(j, &k, &kn) == false || js_take(j, ':') == false) {
            j->bad = true;
            return;
        }
        if (span_is(k, kn, "dtype")) {
            const char *v;
            uint32_t vn;
            if (js_string(j, &v, &vn)) {
                st_dtype(e, v, vn);
                have_dtype = true;
            }
        } else if (span_is(k, kn, "shape")) {
            have_shape = js_take(j, '[');
            e->ndim = 0;
            while (have_shape && j->bad == false && js_take(j, ']') == false) {
                uint64_t v = js_number(j);
                if (e->ndim < MOE_ST_MAX_DIMS) {
                    e->shape[e->ndim] = v;
                    e->ndim += 1;
                } else {
                    j->bad = true;
                }
                js_take(j, ',');
            }
        } else if (span_is(k, kn, "data_offsets")) {
            have_offs = js_take(j, '[');
            e->begin = js_number(j);
            have_offs = have_offs && js_take(j, ',');
            e->end = js_number(j);
            have_offs = have_offs && js_take(j, ']');
        } else {
            js_skip(j);
        }
        js_take(j, ',');
    }
    if (have_dtype == false || have_shape == false || have_offs == false) {
        j->bad = true;
    }
}

/* ---- shards -------------------------------------------------------------------- */

moe_st_file_t moe_st_read(const char *path) {
    moe_st_file_t f;
    memset(&f, 0, sizeof(f));
    int fd = open(path, O_RDONLY);
    if (fd < 0) {
        return f;
    }
    struct stat sb;
    if (fstat(fd, &sb) != 0 || sb.st_size < 8) {
        close(fd);
        return f;
    }
    void *m = mmap(NULL, (size_t)sb.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (m == MAP_FAILED) {
        return f;
    }
    f.bytes = (uint8_t *)m;
    f.mapped = (uint64_t)sb.st_size;
    uint64_t hlen = 0;
    for (uint32_t i = 0; i < 8; i += 1) {
        hlen |= (uint64_t)f.bytes[i] << (8 * i);
    }
    if (hlen > f.mapped - 8) {
        moe_st_free(&f);
        return f;
    }
    f.data = f.bytes + 8 + hlen;
    f.size = f.mapped - 8 - hlen;
    moe_json_t j = {(const char *)f.bytes + 8, (const char *)f.bytes + 8 + hlen, false};
    uint32_t cap = 0;
    if (js_take(&j, '{') == false) {
        j.bad = true;
    }
    while (j.bad == false && js_take(&j, '}') == false) {
        const char *k;
        uint32_t kn;
        if (js_string(&j, &k, &kn) == false || js_take(&j, ':') == false) {
            j.bad = true;
            break;
        }
        if (span_is(k, kn, "__metadata__")) {
            js_skip(&j);
        } else {
            if (f.n == cap) {
                cap = cap == 0 ? 64 : cap * 2;
                moe_st_entry_t *grown = realloc(f.ent, (size_t)cap * sizeof(moe_st_entry_t));
                if (grown == NULL) {
                    j.bad = true;
                    break;
                }
                f.ent = grown;
            }
            moe_st_entry_t *e = &f.ent[f.n];
            memset(e, 0, sizeof(*e));
            e->key = k;
            e->key_len = kn;
            st_entry(&j, e);
            f.n += 1;
        }
        js_take(&j, ',');
    }
    if (j.bad) {
        moe_st_free(&f);
        return f;
    }
    f.ok = true;
    return f;
}

void moe_st_free(moe_st_file_t *f) {
    if (f->bytes != NULL) {
        munmap(f->bytes, (size_t)f->mapped);
    }
    free(f->ent);
    memset(f, 0, sizeof(*f));
}

static const moe_st_entry_t *st_lookup(const moe_st_file_t *f, const char *name) {
    uint32_t n = (uint32_t)strlen(name);
    for (uint32_t i = 0; i < f->n; i += 1) {
        if (f->ent[i].key_len == n && memcmp(f->ent[i].key, name, n) == 0) {
            return &f->ent[i];
        }
    }
    return NULL;
}

bool moe_st_has(const moe_st_file_t *f, const char *name) {
    return f->ok && st_lookup(f, name) != NULL;
}

moe_st_tensor_t moe_st_tensor(const moe_st_file_t *f, const char *name) {
    moe_st_tensor_t t;
    memset(&t, 0, sizeof(t));
    const moe_st_entry_t *e = f->ok ? st_lookup(f, name) : NULL;
    if (e == NULL || e->elem == 0) {
        return t;
    }
    uint64_t rows = 1, cols = 1;
    for (uint32_t i = 0; i < e->ndim; i += 1) { /* leading dimensions fold into rows */
        if (i + 1 < e->ndim) {
            if (e->shape[i] != 0 && rows > UINT64_MAX / e->shape[i]) {
                return t;
            }
            rows *= e->shape[i];
        } else {
            cols = e->shape[i];
        }
    }
    if (cols > UINT32_MAX || (cols != 0 && rows > UINT64_MAX / cols / e->elem)) {
        return t;
    }
    if (e->end < e->begin || e->end > f->size || e->end - e->begin != rows * cols * e->elem) {
        return t;
    }
    t.data = f->data + e->begin;
    t.rows = rows;
    t.cols = (uint32_t)cols;
    t.dtype = e->dtype;
    t.ok = true;
    return t;
}

float moe_st_bf16(const uint8_t *data, uint64_t i) {
    uint32_t bits = ((uint32_t)data[2 * i] | ((uint32_t)data[2 * i + 1] << 8)) << 16;
    float v;
    memcpy(&v, &bits, sizeof(v));
    return v;
}

static int st_name_order(const void *a, const void *b) {
    return strcmp(*(const char *const *)a, *(const char *const *)b);
}

moe_st_set_t moe_st_open_set(const char *dir) {
    moe_st_set_t s = {NULL, 0};
    DIR *d = opendir(dir);
    if (d == NULL) {
        return s;
    }
    char **names = NULL;
    uint32_t n = 0, cap = 0;
    bool ok = true;
    for (struct dirent *de = readdir(d); de != NULL && ok; de = readdir(d)) {
        size_t len = strlen(de->d_name);
        const char *ext = ".safetensors";
        if (len > strlen(ext) && strcmp(de->d_name + len - strlen(ext), ext) == 0) {
            if (n == cap) {
                cap = cap == 0 ? 16 : cap * 2;
                char **grown = realloc(names, (size_t)cap * sizeof(char *));
                if (grown == NULL) {
                    ok = false;
                    break;
                }
                names = grown;
            }
            names[n] = strdup(de->d_name);
            ok = names[n] != NULL;
            n += ok ? 1 : 0;
        }
    }
    closedir(d);
    if (ok && n > 0) {
        qsort(names, n, sizeof(char *), st_name_order); /* shard order = name order */
        s.files = calloc(n, sizeof(moe_st_file_t));
        ok = s.files != NULL;
        for (uint32_t i = 0; i < n && ok; i += 1) {
            char path[4096];
            snprintf(path, sizeof(path), "%s/%s", dir, names[i]);
            s.files[i] = moe_st_read(path);
            ok = s.files[i].ok;
            s.n = i + 1;
        }
    }
    for (uint32_t i = 0; i < n; i += 1) {
        free(names[i]);
    }
    free(names);
    if (ok == false) {
        moe_st_free_set(&s);
    }
    return s;
}

void moe_st_free_set(moe_st_set_t *s) {
    for (uint32_t i = 0; i < s->n; i += 1) {
        moe_st_free(&s->files[i]);
    }
    free(s->files);
    s->files = NULL;
    s->n = 0;
}

moe_st_tensor_t moe_st_find(const moe_st_set_t *s, const char *name) {
    for (uint32_t i = 0; i < s->n; i += 1) {
        if (moe_st_has(&s->files[i], name)) {
            return moe_st_tensor(&s->files[i], name);
        }
    }
    moe_st_tensor_t none;
    memset(&none, 0, sizeof(none));
    return none;
}

/* ---- staging banks ----------------------------------------------------------------- */

static bool stage_open(moe_stage_t *s, moe_cuda_ctx_t *c, uint64_t bytes) {
    s->size = bytes;
    s->used = 0;
    s->host = c != NULL ? moe_cuda_alloc_pinned(c, (size_t)bytes) : malloc((size_t)bytes);
    return s->host != NULL;
}

bool moe_bank_open_slice(moe_bank_t *b, moe_cuda_ctx_t *c, moe_bank_cfg_t cfg, uint32_t local) {
    memset(b, 0, sizeof(*b));
    b->c = c;
    b->pinned = c != NULL;
    uint64_t d = cfg.d, e = cfg.experts, i = cfg.inter, s = cfg.shared, el = local;
    uint64_t dense = ((e + MOE_HOST_PAD_ROWS) * d + 3 * s * d) * sizeof(uint16_t);
    bool ok = stage_open(&b->dense, c, dense);
    ok = ok && stage_open(&b->gu, c, el * 2 * i * d * sizeof(uint16_t));
    ok = ok && stage_open(&b->down, c, el * d * i * sizeof(uint16_t));
    if (ok == false) {
        moe_bank_close(b);
    }
    return ok;
}

bool moe_bank_open(moe_bank_t *b, moe_cuda_ctx_t *c, moe_bank_cfg_t cfg) {
    return moe_bank_open_slice(b, c, cfg, cfg.experts);
}

void moe_bank_close(moe_bank_t *b) {
    moe_stage_t *all[3] = {&b->dense, &b->gu, &b->down};
    for (uint32_t i = 0; i < 3; i += 1) {
        if (all[i]->host != NULL) {
            if (b->pinned) {
                moe_cuda_free_pinned(b->c, all[i]->host);
            } else {
                free(all[i]->host);
            }
        }
    }
    memset(b, 0, sizeof(*b));
}

void moe_bank_reset(moe_bank_t *b) { /* mda_qwen_stage_reset, src/qwen.c:349-354 */
    b->dense.used = 0;
    b->gu.used = 0;
    b->down.used = 0;
    b->moe = 0;
    b->sdown = 0;
    b->fail = false;
}

typedef struct bank_copy_t {
    uint8_t *dst;
    const uint8_t *src;
    uint64_t n;
} bank_copy_t;

static void *bank_copy_run(void *arg) {
    bank_copy_t *j = arg;
    memcpy(j->dst, j->src, (size_t)j->n);
    return NULL;
}

/* Page cache -> staging buffer on several threads (mda_qwen_copy_par, src/qwen.c:283-300):
 * one thread cannot keep up with the host-to-device link on a multi-GB layer. */
static void bank_copy(uint8_t *dst, const uint8_t *src, uint64_t n) {
    if (n < (1u << 20)) {
        memcpy(dst, src, (size_t)n);
        return;
    }
    bank_copy_t jobs[MOE_BANK_THREADS];
    pthread_t th[MOE_BANK_THREADS];
    bool started[MOE_BANK_THREADS];
    uint64_t per = (n + MOE_BANK_THREADS - 1) / MOE_BANK_THREADS;
    for (uint32_t i = 0; i < MOE_BANK_THREADS; i += 1) {
        uint64_t lo = i * per < n ? i * per : n;
        uint64_t hi = lo + per < n ? lo + per : n;
        jobs[i] = (bank_copy_t) {
            .dst = dst + lo,
            .src = src + lo,
            .n = hi - lo,
        };
        started[i] = pthread_create(&th[i], NULL, bank_copy_run, &jobs[i]) == 0;
        if (started[i] == false) {
            bank_copy_run(&jobs[i]);
        }
    }
    for (uint32_t i = 0; i < MOE_BANK_THREADS; i += 1) {
        if (started[i]) {
            pthread_join(th[i], NULL);
        }
    }
}

uint64_t moe_bank_put(moe_bank_t *b, moe_stage_t *s, moe_st_tensor_t t) { /* mda_qwen_put, src/qwen.c:310-321 */
    uint64_t at = s->used;
    if (t.ok == false || t.dtype != MOE_ST_BF16) {
        b->fail = true;
    } else {
        uint64_t bytes = t.rows * t.cols * sizeof(uint16_t);
        if (s->used + bytes > s->size) {
            fprintf(stderr, "moe_bank: staging buffer of %llu bytes is too small\n", (unsigned long long)s->size);
            b->fail = true;
        } else {
            bank_copy((uint8_t *)s->host + at, t.data, bytes);
            s->used += bytes;
        }
    }
    return at / sizeof(uint16_t);
}

void moe_bank_pad_to(moe_bank_t *b, moe_stage_t *s, uint64_t start, uint32_t rows, uint32_t cols) { /* src/qwen.c:330-335 */
    uint64_t want = (start + (uint64_t)rows * cols) * sizeof(uint16_t);
    if (want > s->size) {
        b->fail = true;
    } else if (want > s->used) {
        memset((uint8_t *)s->host + s->used, 0, (size_t)(want - s->used));
        s->used = want;
    }
}

static moe_st_tensor_t bank_find(moe_bank_t *b, const moe_st_set_t *set, const char *prefix, uint32_t l,
                                 const char *suffix, uint64_t rows, uint32_t cols) {
    char name[2 * MOE_ST_MAX_KEY];
    snprintf(name, sizeof(name), "%slayers.%u.%s", prefix, l, suffix); /* mda_qwen_layer_find, src/qwen.c:82-86 */
    moe_st_tensor_t t = moe_st_find(set, name);
    if (t.ok && (t.rows != rows || t.cols != cols)) { /* mda_qwen_shape, src/qwen.c:88-94 */
        fprintf(stderr, "moe_bank: %s is %llu x %u, expected %llu x %u\n", name, (unsigned long long)t.rows, t.cols,
                (unsigned long long)rows, cols);
        t.ok = false;
    }
    if (t.ok == false) {
        b->fail = true;
    }
    return t;
}

/* mda_qwen_put_moe, src/qwen.c:441-452.  The dense stage becomes the operand of the upstream
 * projection: E router rows, the shared gate row, zero rows up to E + 128, then the shared
 * expert's gate and up rows -- so that one product yields the logits, the shared gate logit and
 * the shared expert's pre-activations -- followed by the shared expert's down_proj. */
void moe_bank_put_moe(moe_bank_t *b, const moe_st_set_t *set, const char *prefix, moe_bank_cfg_t cfg, uint32_t l) {
    b->moe = moe_bank_put(b, &b->dense, bank_find(b, set, prefix, l, "mlp.gate.weight", cfg.experts, cfg.d));
    if (cfg.shared != 0) {
        moe_bank_put(b, &b->dense, bank_find(b, set, prefix, l, "mlp.shared_expert_gate.weight", 1, cfg.d));
    }
    moe_bank_pad_to(b, &b->dense, b->moe, cfg.experts + MOE_HOST_PAD_ROWS, cfg.d);
    if (cfg.shared != 0) {
        moe_bank_put(b, &b->dense, bank_find(b, set, prefix, l, "mlp.shared_expert.gate_proj.weight", cfg.shared, cfg.d));
        moe_bank_put(b, &b->dense, bank_find(b, set, prefix, l, "mlp.shared_expert.up_proj.weight", cfg.shared, cfg.d));
        b->sdown = moe_bank_put(b, &b->dense, bank_find(b, set, prefix, l, "mlp.shared_expert.down_proj.weight", cfg.d, cfg.shared));
    }
    moe_bank_put(b, &b->gu, bank_find(b, set, prefix, l, "mlp.experts.gate_up_proj", (uint64_t)cfg.experts * 2 * cfg.inter, cfg.d));
    moe_bank_put(b, &b->down, bank_find(b, set, prefix, l, "mlp.experts.down_proj", (uint64_t)cfg.experts * cfg.d, cfg.inter));
}

/* rows [lo, hi) of a tensor */
static moe_st_tensor_t bank_rows(moe_st_tensor_t t, uint64_t lo, uint64_t hi) {
    if (t.ok && lo <= hi && hi <= t.rows) {
        t.data += lo * t.cols * sizeof(uint16_t);
        t.rows = hi - lo;
    } else {
        t.ok = false;
    }
    return t;
}

void moe_bank_put_moe_slice(moe_bank_t *b, const moe_st_set_t *set, const char *prefix, moe_bank_cfg_t cfg, uint32_t l,
                            uint32_t e_lo, uint32_t e_hi) {
    if (e_lo > e_hi || e_hi > cfg.experts) {
        fprintf(stderr, "moe_bank: expert slice %u..%u outside 0..%u\n", e_lo, e_hi, cfg.experts);
        b->fail = true;
        return;
    }
    /* replicated part: exactly mda_qwen_put_moe's dense stage */
    b->moe = moe_bank_put(b, &b->dense, bank_find(b, set, prefix, l, "mlp.gate.weight", cfg.experts, cfg.d));
    if (cfg.shared != 0) {
        moe_bank_put(b, &b->dense, bank_find(b, set, prefix, l, "mlp.shared_expert_gate.weight", 1, cfg.d));
    }
    moe_bank_pad_to(b, &b->dense, b->moe, cfg.experts + MOE_HOST_PAD_ROWS, cfg.d);
    if (cfg.shared != 0) {
        moe_bank_put(b, &b->dense, bank_find(b, set, prefix, l, "mlp.shared_expert.gate_proj.weight", cfg.shared, cfg.d));
        moe_bank_put(b, &b->dense, bank_find(b, set, prefix, l, "mlp.shared_expert.up_proj.weight", cfg.shared, cfg.d));
        b->sdown = moe_bank_put(b, &b->dense, bank_find(b, set, prefix, l, "mlp.shared_expert.down_proj.weight", cfg.d, cfg.shared));
    }
    /* sharded part: this rank's rows of the two fused expert tensors */
    moe_st_tensor_t gu = bank_find(b, set, prefix, l, "mlp.experts.gate_up_proj", (uint64_t)cfg.experts * 2 * cfg.inter, cfg.d);
    moe_st_tensor_t dn = bank_find(b, set, prefix, l, "mlp.experts.down_proj", (uint64_t)cfg.experts * cfg.d, cfg.inter);
    moe_bank_put(b, &b->gu, bank_rows(gu, (uint64_t)e_lo * 2 * cfg.inter, (uint64_t)e_hi * 2 * cfg.inter));
    moe_bank_put(b, &b->down, bank_rows(dn, (uint64_t)e_lo * cfg.d, (uint64_t)e_hi * cfg.d));
}

static void bank_send(moe_bank_t *b, const moe_stage_t *s, void *dev, bool convert) {
    if (s->used > 0) {
        moe_cuda_write(b->c, dev, s->host, (size_t)s->used); /* mda_qwen_stage_copy, src/qwen.c:356-362 */
        if (convert) { /* mda_qwen_convert, src/qwen.c:365-378 */
            struct mda_pc_qwen_bf16_t pc = {
                .n = (uint32_t)(s->used / sizeof(uint32_t)),
            };
            moe_cuda_bf16_to_f16(b->c, dev, pc);
        }
    }
}

/* mda_qwen_upload, src/qwen.c:381-394.  The copies are enqueued on the context's stream straight
 * from the page-locked stages: the bank must not be reset before moe_cuda_flush. */
void moe_bank_upload(moe_bank_t *b, void *wd, void *wgu, void *wdown, bool convert_gu) {
    if (b->fail || b->c == NULL) {
        return;
    }
    bank_send(b, &b->dense, wd, true);
    bank_send(b, &b->gu, wgu, convert_gu);
    bank_send(b, &b->down, wdown, true);
}

static void *bank_job_run(void *arg) { /* mda_qwen_load_run, src/qwen.c:488-498 */
    moe_bank_job_t *j = arg;
    moe_bank_reset(j->b);
    if (j->e_lo == 0 && j->e_hi == 0) {
        moe_bank_put_moe(j->b, j->set, j->prefix, j->cfg, j->layer);
    } else {
        moe_bank_put_moe_slice(j->b, j->set, j->prefix, j->cfg, j->layer, j->e_lo, j->e_hi);
    }
    return NULL;
}

void moe_bank_prefetch(moe_bank_job_t *job) { /* mda_qwen_prefetch, src/qwen.c:1101-1108 */
    job->started = pthread_create(&job->th, NULL, bank_job_run, job) == 0;
    if (job->started == false) {
        bank_job_run(job); /* no thread to be had: load here */
    }
}

void moe_bank_join(moe_bank_job_t *job) {
    if (job->started) {
        pthread_join(job->th, NULL);
        job->started = false;
    }
}
