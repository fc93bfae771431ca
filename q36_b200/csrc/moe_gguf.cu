// GGUF in: finds a layer's expert tensors in a GGUF v3 file and uploads them in the split-plane layout.
//
// The role of the reference's reader (gguf.c:129-261: header, metadata, tensor directory, aligned data section),
// of its tensor names (q36_model.c:62-75: blk.N.ffn_{gate,up,down}_exps.weight, ffn_gate_inp[_shexp].weight,
// post_attention_norm.weight) and of the MXFP4 branch of upload() (q36_engine.cu:202-228) for this path.
// Host code only: the file is mapped read-only, the directory is indexed by name, tensor data is never copied
// except by the repack into the staging buffer that goes to the device.
#include <cuda_runtime.h>
#include <errno.h>
#include <fcntl.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace q36 {

enum : uint32_t { GG_F32 = 0, GG_F16 = 1, GG_Q8_0 = 8, GG_Q5_K = 13, GG_Q6_K = 14, GG_BF16 = 30, GG_MXFP4 = 39 };   // q36.h:133-141

// bytes per block / elements per block of the tensor types the engine's model file uses (gguf.c:56-75) + BF16
static uint64_t type_block_bytes(uint32_t t) {
    switch (t) {
        case GG_F32: return 4; case GG_F16: return 2; case GG_BF16: return 2; case GG_Q8_0: return 34;
        case GG_Q5_K: return 176; case GG_Q6_K: return 210; case GG_MXFP4: return 17; default: return 0;
    }
}
static uint64_t type_block_elems(uint32_t t) {
    switch (t) {
        case GG_F32: case GG_F16: case GG_BF16: return 1; case GG_Q8_0: case GG_MXFP4: return 32;
        case GG_Q5_K: case GG_Q6_K: return 256; default: return 0;
    }
}

struct GgufTensor { uint32_t type, n_dims; uint64_t dims[4], offset, nbytes; const uint8_t *data; };
struct GgufMeta { uint32_t type; const uint8_t *data; uint64_t len; };   // scalars and strings only (arrays are skipped)

struct GgufFile {
    int fd = -1;
    uint8_t *map = nullptr;
    size_t size = 0;
    uint32_t alignment = 32;
    std::unordered_map<std::string, GgufTensor> tensors;
    std::unordered_map<std::string, GgufMeta> meta;
    ~GgufFile() {
        if (map) munmap(map, size);
        if (fd >= 0) close(fd);
    }
};

static thread_local char g_err[256] = "";
static int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

// bounds-checked cursor over the mapping
struct Cur {
    const uint8_t *p, *end;
    bool get(void *dst, size_t n) {
        if ((size_t)(end - p) < n) return false;
        if (dst) memcpy(dst, p, n);
        p += n;
        return true;
    }
    bool str(std::string *s, const uint8_t **raw = nullptr, uint64_t *len = nullptr) {
        uint64_t n;
        if (!get(&n, 8) || (uint64_t)(end - p) < n) return false;
        if (s) s->assign((const char *)p, (size_t)n);
        if (raw) *raw = p;
        if (len) *len = n;
        p += n;
        return true;
    }
};
static size_t scalar_bytes(uint32_t t) {   // GGUF metadata value types 0..12 (gguf.h:38-42)
    switch (t) {
        case 0: case 1: case 7: return 1; case 2: case 3: return 2; case 4: case 5: case 6: return 4;
        case 10: case 11: case 12: return 8; default: return 0;
    }
}
static bool skip_value(Cur &c, uint32_t t, GgufMeta *m) {
    m->type = t;
    m->data = c.p;
    if (t == 8) {   // string: keep a pointer to the characters
        const uint8_t *raw; uint64_t n;
        if (!c.str(nullptr, &raw, &n)) return false;
        m->data = raw; m->len = n;
        return true;
    }
    if (t == 9) {   // array: element type, count, elements
        uint32_t et; uint64_t n;
        if (!c.get(&et, 4) || !c.get(&n, 8)) return false;
        if (et == 8) { for (uint64_t i = 0; i < n; i++) if (!c.str(nullptr)) return false; }
        else { const size_t es = scalar_bytes(et); if (!es || n > (uint64_t)(c.end - c.p) / es || !c.get(nullptr, es * n)) return false; }
        m->len = 0;
        return true;
    }
    const size_t es = scalar_bytes(t);
    m->len = es;
    return es && c.get(nullptr, es);
}

static int gguf_open_impl(const char *path, GgufFile **out) {
    GgufFile *g = new GgufFile;
    auto bad = [&](int code) { delete g; return code; };
    g->fd = open(path, O_RDONLY);
    if (g->fd < 0) return bad(fail(Q36_MOE_EIO, "open %s: %s", path, strerror(errno)));
    struct stat st;
    if (fstat(g->fd, &st) != 0) return bad(fail(Q36_MOE_EIO, "fstat %s: %s", path, strerror(errno)));
    g->size = (size_t)st.st_size;
    if (g->size < 24) return bad(fail(Q36_MOE_EIO, "%s: too short for a GGUF header", path));
    void *m = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) return bad(fail(Q36_MOE_EIO, "mmap %s: %s", path, strerror(errno)));
    g->map = (uint8_t *)m;
    madvise(g->map, g->size, MADV_SEQUENTIAL);   // the file is streamed once towards the device
    Cur c{g->map, g->map + g->size};
    uint8_t magic[4];
    uint32_t version = 0;
    uint64_t n_tensors = 0, n_kv = 0;
    if (!c.get(magic, 4) || memcmp(magic, "GGUF", 4)) return bad(fail(Q36_MOE_EIO, "%s: not a GGUF file", path));
    if (!c.get(&version, 4) || version != 3) return bad(fail(Q36_MOE_EIO, "%s: GGUF version %u (only 3 is read)", path, version));
    if (!c.get(&n_tensors, 8) || !c.get(&n_kv, 8)) return bad(fail(Q36_MOE_EIO, "%s: truncated header", path));
    for (uint64_t i = 0; i < n_kv; i++) {
        std::string key;
        uint32_t t;
        GgufMeta mv{};
        if (!c.str(&key) || !c.get(&t, 4) || !skip_value(c, t, &mv)) return bad(fail(Q36_MOE_EIO, "%s: bad metadata entry %llu", path, (unsigned long long)i));
        if (t != 9) g->meta.emplace(std::move(key), mv);
    }
    std::vector<std::pair<std::string, GgufTensor>> dir;
    for (uint64_t i = 0; i < n_tensors; i++) {
        std::string name;
        GgufTensor t{};
        if (!c.str(&name) || !c.get(&t.n_dims, 4) || t.n_dims > 4) return bad(fail(Q36_MOE_EIO, "%s: bad tensor entry %llu", path, (unsigned long long)i));
        for (uint32_t d = 0; d < 4; d++) t.dims[d] = 1;
        for (uint32_t d = 0; d < t.n_dims; d++) if (!c.get(&t.dims[d], 8)) return bad(fail(Q36_MOE_EIO, "%s: truncated tensor dims", path));
        if (!c.get(&t.type, 4) || !c.get(&t.offset, 8)) return bad(fail(Q36_MOE_EIO, "%s: truncated tensor entry", path));
        dir.emplace_back(std::move(name), t);
    }
    auto al = g->meta.find("general.alignment");
    if (al != g->meta.end() && al->second.len >= 4) { uint32_t a; memcpy(&a, al->second.data, 4); if (a) g->alignment = a; }
    const size_t here = (size_t)(c.p - g->map);
    const uint8_t *base = g->map + (here + g->alignment - 1) / g->alignment * g->alignment;
    for (auto &e : dir) {
        GgufTensor &t = e.second;
        uint64_t nelem = 1;
        for (uint32_t d = 0; d < t.n_dims; d++) nelem *= t.dims[d];
        const uint64_t bb = type_block_bytes(t.type), be = type_block_elems(t.type);
        t.nbytes = (bb && be) ? nelem / be * bb : 0;
        t.data = base + t.offset;
        if (t.data < base || t.data + t.nbytes > g->map + g->size) return bad(fail(Q36_MOE_EIO, "%s: tensor %s runs past the end of the file", path, e.first.c_str()));
        g->tensors.emplace(std::move(e.first), t);
    }
    *out = g;
    return Q36_MOE_OK;
}

static const GgufTensor *find(const GgufFile *g, const char *fmt, int layer, char *name_out = nullptr) {
    char name[160];
    snprintf(name, sizeof name, fmt, layer);
    if (name_out) strcpy(name_out, name);
    auto it = g->tensors.find(name);
    return it == g->tensors.end() ? nullptr : &it->second;
}

// f32 / bf16 / f16 tensor values widened to f32 (the engine widens BF16 router tensors at upload, q36_model.c:57-61)
static int widen_to_f32(const GgufTensor *t, float *dst, uint64_t n) {
    if (t->type == GG_F32) { memcpy(dst, t->data, n * 4); return Q36_MOE_OK; }
    if (t->type == GG_BF16) {
        const uint16_t *s = (const uint16_t *)t->data;
        for (uint64_t i = 0; i < n; i++) { const uint32_t u = (uint32_t)s[i] << 16; memcpy(dst + i, &u, 4); }
        return Q36_MOE_OK;
    }
    return Q36_MOE_EUNSUPPORTED;
}

}  // namespace q36

using namespace q36;

extern "C" {

const char *q36_gguf_last_error(void) { return g_err; }

int q36_gguf_open(const char *path, void **gguf_out) {
    if (!path || !gguf_out) return Q36_MOE_EINVAL;
    GgufFile *g = nullptr;
    const int rc = gguf_open_impl(path, &g);
    if (rc == Q36_MOE_OK) *gguf_out = g;
    return rc;
}

int q36_gguf_close(void *gguf) {
    if (!gguf) return Q36_MOE_EINVAL;
    delete (GgufFile *)gguf;
    return Q36_MOE_OK;
}

int q36_gguf_tensor(const void *gguf, const char *name, int *ggml_type, int *n_dims, uint64_t *dims4, const void **host_data,
                    uint64_t *nbytes) {
    const GgufFile *g = (const GgufFile *)gguf;
    if (!g || !name) return Q36_MOE_EINVAL;
    auto it = g->tensors.find(name);
    if (it == g->tensors.end()) return fail(Q36_MOE_EIO, "tensor %s not in the file", name);
    const GgufTensor &t = it->second;
    if (ggml_type) *ggml_type = (int)t.type;
    if (n_dims) *n_dims = (int)t.n_dims;
    if (dims4) for (int d = 0; d < 4; d++) dims4[d] = t.dims[d];
    if (host_data) *host_data = t.data;
    if (nbytes) *nbytes = t.nbytes;
    return Q36_MOE_OK;
}

int q36_gguf_meta_u32(const void *gguf, const char *key, uint32_t *out) {
    const GgufFile *g = (const GgufFile *)gguf;
    if (!g || !key || !out) return Q36_MOE_EINVAL;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return fail(Q36_MOE_EIO, "metadata key %s not in the file", key);
    const GgufMeta &m = it->second;
    if ((m.type == 4 || m.type == 5) && m.len == 4) { memcpy(out, m.data, 4); return Q36_MOE_OK; }
    if ((m.type == 10 || m.type == 11) && m.len == 8) { uint64_t v; memcpy(&v, m.data, 8); *out = (uint32_t)v; return Q36_MOE_OK; }
    return fail(Q36_MOE_EUNSUPPORTED, "metadata key %s is not an integer", key);
}

int q36_moe_gguf_layer_shape(const void *gguf, int layer, int *n_expert, int *D, int *FF, int *ggml_types3) {
    const GgufFile *g = (const GgufFile *)gguf;
    if (!g || layer < 0) return Q36_MOE_EINVAL;
    static const char *fmts[3] = {"blk.%d.ffn_gate_exps.weight", "blk.%d.ffn_up_exps.weight", "blk.%d.ffn_down_exps.weight"};
    const GgufTensor *t[3];
    char name[160];
    for (int i = 0; i < 3; i++) {
        t[i] = find(g, fmts[i], layer, name);
        if (!t[i]) return fail(Q36_MOE_EIO, "tensor %s not in the file", name);
        if (t[i]->n_dims != 3) return fail(Q36_MOE_EUNSUPPORTED, "tensor %s has %u dimensions, expected [K, M, experts]", name, t[i]->n_dims);
        if (ggml_types3) ggml_types3[i] = (int)t[i]->type;
    }
    // gate/up: [K = D, M = FF, E]; down: [K = FF, M = D, E] (q36_model.h:75-77)
    const uint64_t d = t[0]->dims[0], ff = t[0]->dims[1], e = t[0]->dims[2];
    if (t[1]->dims[0] != d || t[1]->dims[1] != ff || t[1]->dims[2] != e || t[2]->dims[0] != ff || t[2]->dims[1] != d || t[2]->dims[2] != e)
        return fail(Q36_MOE_EUNSUPPORTED, "layer %d: gate/up/down expert tensor shapes do not agree", layer);
    if (n_expert) *n_expert = (int)e;
    if (D) *D = (int)d;
    if (FF) *FF = (int)ff;
    return Q36_MOE_OK;
}

int q36_moe_gguf_upload_layer(const void *gguf, int layer, int e0, int e1, void *dev_Wg, void *dev_Wu, void *dev_Wd) {
    const GgufFile *g = (const GgufFile *)gguf;
    int E, D, FF, types[3];
    int rc = q36_moe_gguf_layer_shape(gguf, layer, &E, &D, &FF, types);
    if (rc) return rc;
    if (!dev_Wg || !dev_Wu || !dev_Wd || e0 < 0 || e1 <= e0 || e1 > E) return Q36_MOE_EINVAL;
    for (int i = 0; i < 3; i++)
        if (types[i] != (int)GG_MXFP4)
            return fail(Q36_MOE_EUNSUPPORTED, "layer %d: expert tensor %d has ggml type %d; only MXFP4 (39) is taken by this path", layer, i, types[i]);
    static const char *fmts[3] = {"blk.%d.ffn_gate_exps.weight", "blk.%d.ffn_up_exps.weight", "blk.%d.ffn_down_exps.weight"};
    void *dst[3] = {dev_Wg, dev_Wu, dev_Wd};
    for (int i = 0; i < 3; i++) {
        const GgufTensor *t = find(g, fmts[i], layer);
        if ((rc = q36_moe_upload_mxfp4(t->data, (int)t->dims[0], (int)t->dims[1], e0, e1, dst[i]))) return rc;
    }
    return Q36_MOE_OK;
}

int q36_moe_gguf_upload_shared(const void *gguf, int layer, void *dev_Sg, void *dev_Su, void *dev_Sd) {
    const GgufFile *g = (const GgufFile *)gguf;
    if (!g || layer < 0 || !dev_Sg || !dev_Su || !dev_Sd) return Q36_MOE_EINVAL;
    static const char *fmts[3] = {"blk.%d.ffn_gate_shexp.weight", "blk.%d.ffn_up_shexp.weight", "blk.%d.ffn_down_shexp.weight"};
    void *dst[3] = {dev_Sg, dev_Su, dev_Sd};
    char name[160];
    for (int i = 0; i < 3; i++) {
        const GgufTensor *t = find(g, fmts[i], layer, name);
        if (!t) return fail(Q36_MOE_EIO, "tensor %s not in the file", name);
        if (t->type != GG_MXFP4)   // the published model keeps the shared expert in Q8_0 (q36_model.c:73-75): not this path
            return fail(Q36_MOE_EUNSUPPORTED, "tensor %s has ggml type %u; only MXFP4 (39) is taken by this path", name, t->type);
        if (t->n_dims != 2) return fail(Q36_MOE_EUNSUPPORTED, "tensor %s has %u dimensions, expected [K, M]", name, t->n_dims);
        const int rc = q36_moe_upload_mxfp4(t->data, (int)t->dims[0], (int)t->dims[1], 0, 1, dst[i]);
        if (rc) return rc;
    }
    return Q36_MOE_OK;
}

int q36_moe_gguf_upload_router(const void *gguf, int layer, float *dev_router) {
    const GgufFile *g = (const GgufFile *)gguf;
    if (!g || layer < 0 || !dev_router) return Q36_MOE_EINVAL;
    char name[160];
    const GgufTensor *r = find(g, "blk.%d.ffn_gate_inp.weight", layer, name);
    if (!r) return fail(Q36_MOE_EIO, "tensor %s not in the file", name);
    if (r->n_dims != 2) return fail(Q36_MOE_EUNSUPPORTED, "tensor %s has %u dimensions, expected [D, experts]", name, r->n_dims);
    const uint64_t D = r->dims[0], E = r->dims[1];
    const GgufTensor *s = find(g, "blk.%d.ffn_gate_inp_shexp.weight", layer, name);
    if (!s) return fail(Q36_MOE_EIO, "tensor %s not in the file", name);
    uint64_t sn = 1;
    for (uint32_t d = 0; d < s->n_dims; d++) sn *= s->dims[d];
    if (sn != D) return fail(Q36_MOE_EUNSUPPORTED, "tensor %s has %llu elements, expected %llu", name, (unsigned long long)sn, (unsigned long long)D);
    std::vector<float> host((E + 1) * D);
    int rc;
    if ((rc = widen_to_f32(r, host.data(), E * D)) || (rc = widen_to_f32(s, host.data() + E * D, D)))
        return fail(rc, "layer %d: router tensors must be F32 or BF16", layer);
    const cudaError_t e = cudaMemcpy(dev_router, host.data(), host.size() * 4, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { last_cuda_error() = (int)e; return Q36_MOE_ECUDA; }
    return Q36_MOE_OK;
}

int q36_moe_gguf_upload_f32(const void *gguf, const char *name, float *dev_dst, uint64_t n) {
    const GgufFile *g = (const GgufFile *)gguf;
    if (!g || !name || !dev_dst) return Q36_MOE_EINVAL;
    auto it = g->tensors.find(name);
    if (it == g->tensors.end()) return fail(Q36_MOE_EIO, "tensor %s not in the file", name);
    const GgufTensor &t = it->second;
    uint64_t ne = 1;
    for (uint32_t d = 0; d < t.n_dims; d++) ne *= t.dims[d];
    if (ne != n) return fail(Q36_MOE_EINVAL, "tensor %s has %llu elements, caller expects %llu", name, (unsigned long long)ne, (unsigned long long)n);
    std::vector<float> host(n);
    const int rc = widen_to_f32(&t, host.data(), n);
    if (rc) return fail(rc, "tensor %s must be F32 or BF16", name);
    const cudaError_t e = cudaMemcpy(dev_dst, host.data(), n * 4, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { last_cuda_error() = (int)e; return Q36_MOE_ECUDA; }
    return Q36_MOE_OK;
}

}  // extern "C"
