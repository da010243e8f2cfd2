/* Expert-weight loader for converted Clef-Omni checkpoints (GGUF v3).
 *
 * Maps the file, walks its header and binds, per decoder layer, the tensors the MoE block
 * consumes, with the checks the reference's engine applies when it binds the same tensors
 * (clef.c:194-205 `bind_experts`, clef.c:232-246 the per-layer names; tools/convert_omni.py:135-139
 * writes them):
 *
 *   blk.N.ffn_norm.weight           F32   [H]
 *   blk.N.ffn_router.weight         BF16  [H, E]            (ne[0] is the row length)
 *   blk.N.ffn_gate_up_exps.weight   BF16  [H, 2*ffn, E]     gate rows then up rows per expert
 *   blk.N.ffn_down_exps.weight      BF16  [ffn, H, E]
 *   clef.attention.layer_norm_rms_epsilon   F32 key (must be 1e-6), and the keys that pin the
 *   geometry: general.architecture, clef.block_count, clef.embedding_length,
 *   clef.feed_forward_length, clef.moe.expert_count, clef.moe.expert_used_count,
 *   clef.moe.normalize_topk (clef.c:27-36, 76-90)
 *
 * The reader is a plain restatement of the published container format: little-endian header
 * (magic "GGUF", version 3, tensor count, key/value count), key/value pairs, tensor infos
 * (name, rank, extents, element type, offset into the data section), data section aligned to
 * `general.alignment` (default 32).  Every length is checked against the file size before use.
 */
#define _GNU_SOURCE
#include <fcntl.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "../../include/clef_cuda_omni.h"

enum { T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STRING, T_ARRAY, T_U64, T_I64, T_F64, T_COUNT };
enum { GG_F32 = 0, GG_F16 = 1, GG_BF16 = 30 };

typedef struct {
    const char *name; uint64_t name_len;
    uint32_t n_dims, type;
    uint64_t ne[4];
    uint64_t offset, nbytes;      /* offset is absolute in the file */
} tensor_info;

typedef struct {
    int fd;
    const uint8_t *base;
    uint64_t size, pos;
    uint64_t n_tensors;
    tensor_info *tensors;
    float rms_eps; bool have_eps;
    uint32_t alignment;
    /* the configuration keys that fix the block's geometry (clef.c:34-36, 76-79), 0 = absent */
    uint32_t cfg_H, cfg_ffn, cfg_experts, cfg_used, cfg_layers;
    int normalize_topk;           /* -1 absent, else the stored bool */
    bool arch_clef;
    char err[256];
} gguf_view;

static bool fail(gguf_view *v, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(v->err, sizeof v->err, fmt, ap);
    va_end(ap);
    return false;
}

static bool need(gguf_view *v, uint64_t n) {
    if (n > v->size || v->pos > v->size - n) return fail(v, "gguf: truncated file (offset %llu)", (unsigned long long)v->pos);
    return true;
}
static bool rd_u32(gguf_view *v, uint32_t *out) { if (!need(v, 4)) return false; memcpy(out, v->base + v->pos, 4); v->pos += 4; return true; }
static bool rd_u64(gguf_view *v, uint64_t *out) { if (!need(v, 8)) return false; memcpy(out, v->base + v->pos, 8); v->pos += 8; return true; }
static bool rd_str(gguf_view *v, const char **p, uint64_t *len) {
    if (!rd_u64(v, len) || !need(v, *len)) return false;
    *p = (const char *)(v->base + v->pos);
    v->pos += *len;
    return true;
}

static const uint64_t scalar_size[T_COUNT] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};

static bool skip_value(gguf_view *v, uint32_t type, int depth) {
    if (type >= T_COUNT) return fail(v, "gguf: unknown value type %u", type);
    if (type == T_STRING) { const char *p; uint64_t n; return rd_str(v, &p, &n); }
    if (type == T_ARRAY) {
        uint32_t et; uint64_t count;
        if (depth > 2) return fail(v, "gguf: arrays nested too deep");
        if (!rd_u32(v, &et) || !rd_u64(v, &count)) return false;
        if (et >= T_COUNT) return fail(v, "gguf: unknown array element type %u", et);
        if (et != T_STRING && et != T_ARRAY) {
            if (count > v->size / scalar_size[et]) return fail(v, "gguf: array longer than the file");
            if (!need(v, count * scalar_size[et])) return false;
            v->pos += count * scalar_size[et];
            return true;
        }
        for (uint64_t i = 0; i < count; i++) if (!skip_value(v, et, depth + 1)) return false;
        return true;
    }
    if (!need(v, scalar_size[type])) return false;
    v->pos += scalar_size[type];
    return true;
}

static bool key_is(const char *p, uint64_t n, const char *lit) { return n == strlen(lit) && !memcmp(p, lit, n); }

static void view_close(gguf_view *v) {
    free(v->tensors);
    if (v->base) munmap((void *)v->base, v->size);
    if (v->fd >= 0) close(v->fd);
    v->tensors = NULL; v->base = NULL; v->fd = -1;
}

static bool view_open(gguf_view *v, const char *path) {
    memset(v, 0, sizeof *v);
    v->fd = -1;
    v->alignment = 32;
    v->normalize_topk = -1;
    if (!path) return fail(v, "gguf: no path");
    v->fd = open(path, O_RDONLY);
    if (v->fd < 0) return fail(v, "gguf: cannot open %s", path);
    struct stat st;
    if (fstat(v->fd, &st) != 0 || st.st_size < 24) return fail(v, "gguf: %s is too short", path);
    v->size = (uint64_t)st.st_size;
    void *m = mmap(NULL, v->size, PROT_READ, MAP_PRIVATE, v->fd, 0);
    if (m == MAP_FAILED) return fail(v, "gguf: cannot map %s", path);
    v->base = m;
    uint32_t magic, version; uint64_t n_kv;
    if (!rd_u32(v, &magic) || !rd_u32(v, &version) || !rd_u64(v, &v->n_tensors) || !rd_u64(v, &n_kv)) return false;
    if (magic != 0x46554747u) return fail(v, "gguf: bad magic");
    if (version != 3) return fail(v, "gguf: unsupported version %u", version);
    if (v->n_tensors > v->size / 32 || n_kv > v->size / 12) return fail(v, "gguf: counts larger than the file");
    for (uint64_t i = 0; i < n_kv; i++) {
        const char *k; uint64_t kn; uint32_t type;
        if (!rd_str(v, &k, &kn) || !rd_u32(v, &type)) return false;
        uint32_t *u32_dst = NULL;
        if (type == T_U32) {
            if (key_is(k, kn, "clef.embedding_length")) u32_dst = &v->cfg_H;
            else if (key_is(k, kn, "clef.feed_forward_length")) u32_dst = &v->cfg_ffn;
            else if (key_is(k, kn, "clef.moe.expert_count")) u32_dst = &v->cfg_experts;
            else if (key_is(k, kn, "clef.moe.expert_used_count")) u32_dst = &v->cfg_used;
            else if (key_is(k, kn, "clef.block_count")) u32_dst = &v->cfg_layers;
        }
        if (u32_dst) {
            if (!need(v, 4)) return false;
            memcpy(u32_dst, v->base + v->pos, 4);
        } else if (type == T_BOOL && key_is(k, kn, "clef.moe.normalize_topk")) {
            if (!need(v, 1)) return false;
            v->normalize_topk = v->base[v->pos];
        } else if (type == T_STRING && key_is(k, kn, "general.architecture")) {
            uint64_t n;
            if (!need(v, 8)) return false;
            memcpy(&n, v->base + v->pos, 8);
            v->arch_clef = n == 4 && v->size - v->pos >= 12 && !memcmp(v->base + v->pos + 8, "clef", 4);
        }
        if (type == T_F32 && key_is(k, kn, "clef.attention.layer_norm_rms_epsilon")) {
            if (!need(v, 4)) return false;
            memcpy(&v->rms_eps, v->base + v->pos, 4);
            v->have_eps = true;
        } else if (type == T_U32 && key_is(k, kn, "general.alignment")) {
            if (!need(v, 4)) return false;
            memcpy(&v->alignment, v->base + v->pos, 4);
            if (v->alignment == 0 || (v->alignment & (v->alignment - 1))) return fail(v, "gguf: alignment is not a power of two");
        }
        if (!skip_value(v, type, 0)) return false;
    }
    v->tensors = calloc(v->n_tensors ? v->n_tensors : 1, sizeof *v->tensors);
    if (!v->tensors) return fail(v, "gguf: out of memory");
    for (uint64_t i = 0; i < v->n_tensors; i++) {
        tensor_info *t = &v->tensors[i];
        if (!rd_str(v, &t->name, &t->name_len) || !rd_u32(v, &t->n_dims)) return false;
        if (t->n_dims < 1 || t->n_dims > 4) return fail(v, "gguf: tensor rank %u", t->n_dims);
        uint64_t count = 1;
        for (int d = 0; d < 4; d++) t->ne[d] = 1;
        for (uint32_t d = 0; d < t->n_dims; d++) {
            if (!rd_u64(v, &t->ne[d])) return false;
            if (t->ne[d] == 0 || count > v->size / t->ne[d]) return fail(v, "gguf: tensor %.*s larger than the file", (int)t->name_len, t->name);
            count *= t->ne[d];
        }
        if (!rd_u32(v, &t->type) || !rd_u64(v, &t->offset)) return false;
        const uint64_t esz = t->type == GG_F32 ? 4 : (t->type == GG_F16 || t->type == GG_BF16) ? 2 : 0;
        t->nbytes = count * esz;          /* 0 for element types this loader never binds */
    }
    const uint64_t a = v->alignment;
    const uint64_t data = (v->pos + a - 1) / a * a;
    if (data > v->size) return fail(v, "gguf: truncated file (no data section)");
    const uint64_t avail = v->size - data;
    for (uint64_t i = 0; i < v->n_tensors; i++) {
        tensor_info *t = &v->tensors[i];
        if (t->offset % a) return fail(v, "gguf: tensor %.*s is not aligned", (int)t->name_len, t->name);
        if (t->offset > avail || t->nbytes > avail - t->offset)
            return fail(v, "gguf: tensor %.*s runs past the end of the file", (int)t->name_len, t->name);
        t->offset += data;
    }
    return true;
}

static const tensor_info *find(const gguf_view *v, const char *name) {
    const size_t n = strlen(name);
    for (uint64_t i = 0; i < v->n_tensors; i++)
        if (v->tensors[i].name_len == n && !memcmp(v->tensors[i].name, name, n)) return &v->tensors[i];
    return NULL;
}

/* clef.c:194-205: type, rank and every extent must match */
static const tensor_info *want(gguf_view *v, const char *name, uint32_t type, uint32_t n_dims, uint64_t ne0, uint64_t ne1,
                               uint64_t ne2) {
    const tensor_info *t = find(v, name);
    if (!t || t->type != type || t->n_dims != n_dims || t->ne[0] != ne0 || t->ne[1] != ne1 || t->ne[2] != ne2 || t->ne[3] != 1) {
        fail(v, n_dims == 3 ? "model: missing or invalid rank-3 expert tensor %s" : "model: missing or invalid tensor %s", name);
        return NULL;
    }
    return t;
}

typedef struct { const tensor_info *norm, *router, *gate_up, *down; } layer_tensors;

static bool layer_find(gguf_view *v, int l, uint64_t H, uint64_t ffn, uint64_t E, layer_tensors *out) {
    char name[96];
    snprintf(name, sizeof name, "blk.%d.ffn_norm.weight", l);
    if (!(out->norm = want(v, name, GG_F32, 1, H, 1, 1))) return false;
    snprintf(name, sizeof name, "blk.%d.ffn_router.weight", l);
    if (!(out->router = want(v, name, GG_BF16, 2, H, E, 1))) return false;
    snprintf(name, sizeof name, "blk.%d.ffn_gate_up_exps.weight", l);
    if (!(out->gate_up = want(v, name, GG_BF16, 3, H, 2 * ffn, E))) return false;
    snprintf(name, sizeof name, "blk.%d.ffn_down_exps.weight", l);
    if (!(out->down = want(v, name, GG_BF16, 3, ffn, H, E))) return false;
    return true;
}

/* The reference treats the metadata as untrusted and pins the geometry before it touches a
 * tensor (clef.c:16-24 `cfg_u32`, clef.c:27-32 the architecture, clef.c:55-57 the epsilon,
 * clef.c:76-90 the Omni geometry and routing configuration); same order and messages here for
 * the keys the block depends on.  top_k = 0 accepts any count from 1 to the expert count. */
static bool config_ok(gguf_view *v, int n_layer, uint64_t H, uint64_t ffn, uint64_t E, uint64_t top_k) {
    if (!v->arch_clef) return fail(v, "model: not a clef GGUF (convert with tools/convert.py)");
    const struct { const char *key; uint32_t value; } need_u32[] = {
        {"clef.block_count", v->cfg_layers}, {"clef.embedding_length", v->cfg_H}, {"clef.feed_forward_length", v->cfg_ffn},
    };
    for (size_t i = 0; i < sizeof need_u32 / sizeof need_u32[0]; i++)
        if (need_u32[i].value == 0 || need_u32[i].value > (1u << 24)) return fail(v, "model: missing or invalid %s", need_u32[i].key);
    if (!v->have_eps) return fail(v, "model: missing rms eps / rope base");
    if (v->cfg_experts == 0 || v->cfg_experts > (1u << 24)) return fail(v, "model: missing or invalid clef.moe.expert_count");
    if (v->cfg_used == 0 || v->cfg_used > (1u << 24)) return fail(v, "model: missing or invalid clef.moe.expert_used_count");
    if (v->cfg_H != H || v->cfg_ffn != ffn || v->cfg_experts != E || v->cfg_used > v->cfg_experts ||
        (top_k && v->cfg_used != top_k) || v->rms_eps != 1e-6f || v->normalize_topk != 1)
        return fail(v, "model: unsupported Omni decoder/head geometry or routing configuration");
    if (n_layer < 1 || (uint64_t)n_layer > v->cfg_layers) return fail(v, "model: the checkpoint has %u layers", v->cfg_layers);
    return true;
}

static void copy_err(const gguf_view *v, char *err, size_t errlen) {
    if (err && errlen) snprintf(err, errlen, "%s", v->err);
}

bool clef_omni_gguf_check(const char *path, int n_layer, int H, int ffn, int n_expert, float *rms_eps, char *err,
                          size_t errlen) {
    gguf_view v;
    bool ok = view_open(&v, path);
    if (ok && (n_layer < 1 || H < 1 || ffn < 1 || n_expert < 1)) ok = fail(&v, "model: invalid Omni dimensions");
    if (ok) ok = config_ok(&v, n_layer, (uint64_t)H, (uint64_t)ffn, (uint64_t)n_expert, 0);
    for (int l = 0; ok && l < n_layer; l++) {
        layer_tensors t;
        ok = layer_find(&v, l, (uint64_t)H, (uint64_t)ffn, (uint64_t)n_expert, &t);
    }
    if (ok && rms_eps) *rms_eps = v.rms_eps;
    if (!ok) copy_err(&v, err, errlen);
    view_close(&v);
    return ok;
}

bool clef_omni_bind_gguf(clef_gpu *g, const char *path, int n_layer, char *err, size_t errlen) {
    gguf_view v;
    bool ok = view_open(&v, path);
    if (ok && (!g || n_layer < 1)) ok = fail(&v, "cuda: invalid Omni expert tensor binding");
    if (ok) ok = config_ok(&v, n_layer, 2048, 768, 128, 8);
    if (!ok) { copy_err(&v, err, errlen); view_close(&v); return false; }
    for (int l = 0; ok && l < n_layer; l++) {
        layer_tensors t;
        /* the block is built for exactly these extents (clef.c:78-90 pins them for the Omni backbone) */
        ok = layer_find(&v, l, 2048, 768, 128, &t);
        if (!ok) { copy_err(&v, err, errlen); break; }
        ok = clef_omni_bind_layer(g, l, v.base + t.router->offset, v.base + t.gate_up->offset, v.base + t.down->offset, NULL,
                                  CLEF_OMNI_HOST, err, errlen) &&
             clef_omni_bind_norm(g, l, (const float *)(v.base + t.norm->offset), v.rms_eps, CLEF_OMNI_HOST, err, errlen);
    }
    view_close(&v);          /* the device holds its own copy; nothing points into the mapping any more */
    return ok;
}
