// Test harness for the ggml backend plugin (libggml-ameva-b200.so). It stands in for the host application: a minimal
// ggml-base (the functions the plugin calls, restated for the tensor types and ops of the tests) and a driver that walks
// the plugin's tables the way ggml's loader, allocator and scheduler do. Built against the host's ggml headers; not part
// of the product.
//
//   driver probe                                   registry / device / buffer-type facts and the ABI self-check, no device
//   driver mulmat <type> <M> <N> <K> <w.bin> <x.bin> <y.bin>
//                                                  uploads ggml blocks + f32 activations, runs a one-node MUL_MAT graph,
//                                                  writes y; also checks weight read-back (whole, partial), a partial
//                                                  set_tensor, and that a graph with an unsupported node is refused
//   driver layer <type> <K> <Nq> <Nkv> <Nff> <M2> <dir>
//                                                  a decoder-layer-shaped graph of one activation row (q / k / v sharing
//                                                  src1, o + residual ADD, gate / up + SWIGLU, RMS_NORM + MUL, a row-range
//                                                  view of a weight) followed by a graph with M2 activation rows that
//                                                  needs larger scratch; counters, host-side failure injection, teardown.
//                                                  Inputs are read from <dir>, outputs written there.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "ggml-backend-impl.h"
#include "ggml-backend.h"
#include "ggml.h"

#include "../../include/ggml_ameva_b200.h"

struct ggml_cgraph {
    int n_nodes;
    ggml_tensor** nodes;
};

static void traits(enum ggml_type t, size_t* type_size, int64_t* blck) {
    switch (t) {
        case GGML_TYPE_F32: *type_size = 4; *blck = 1; break;
        case GGML_TYPE_Q4_0: *type_size = 18; *blck = 32; break;
        case GGML_TYPE_Q8_0: *type_size = 34; *blck = 32; break;
        case GGML_TYPE_Q4_K: *type_size = 144; *blck = 256; break;
        case GGML_TYPE_Q6_K: *type_size = 210; *blck = 256; break;
        case GGML_TYPE_Q5_K: *type_size = 176; *blck = 256; break;
        case GGML_TYPE_IQ4_XS: *type_size = 136; *blck = 256; break;
        case GGML_TYPE_Q3_K: *type_size = 110; *blck = 256; break;
        case GGML_TYPE_Q2_K: *type_size = 84; *blck = 256; break;
        case GGML_TYPE_Q4_1: *type_size = 20; *blck = 32; break;
        case GGML_TYPE_Q5_1: *type_size = 24; *blck = 32; break;
        case GGML_TYPE_Q5_0: *type_size = 22; *blck = 32; break;
        case GGML_TYPE_IQ4_NL: *type_size = 18; *blck = 32; break;
        case GGML_TYPE_F16: *type_size = 2; *blck = 1; break;
        case GGML_TYPE_I32: *type_size = 4; *blck = 1; break;
        case GGML_TYPE_I64: *type_size = 8; *blck = 1; break;
        default: fprintf(stderr, "shim: type %d not in the test set\n", (int)t); abort();
    }
}

// ---- the stand-in for ggml-base ---------------------------------------------------------------------------------------
struct ggml_context {
    std::vector<ggml_tensor*> tensors;
};

extern "C" {
size_t ggml_nbytes(const ggml_tensor* t) {
    size_t ts;
    int64_t bs;
    traits(t->type, &ts, &bs);
    if (bs == 1) {   // as ggml: the span from the first to the last element, whatever the strides
        size_t n = ts;
        for (int i = 0; i < 4; ++i) n += (size_t)(t->ne[i] - 1) * t->nb[i];
        return n;
    }
    return (size_t)(t->ne[0] / bs) * ts * (size_t)(t->ne[1] * t->ne[2] * t->ne[3]);
}
bool ggml_is_contiguous(const ggml_tensor* t) {
    size_t ts;
    int64_t bs;
    traits(t->type, &ts, &bs);
    return t->nb[0] == ts && t->nb[1] == ts * (size_t)(t->ne[0] / bs) && t->nb[2] == t->nb[1] * (size_t)t->ne[1] &&
           t->nb[3] == t->nb[2] * (size_t)t->ne[2];
}
bool ggml_is_empty(const ggml_tensor* t) { return t->ne[0] == 0 || t->ne[1] == 0 || t->ne[2] == 0 || t->ne[3] == 0; }
const char* ggml_op_name(enum ggml_op op) {
    switch (op) {
        case GGML_OP_NONE: return "NONE";
        case GGML_OP_ADD: return "ADD";
        case GGML_OP_MUL: return "MUL";
        case GGML_OP_RMS_NORM: return "RMS_NORM";
        case GGML_OP_MUL_MAT: return "MUL_MAT";
        case GGML_OP_RESHAPE: return "RESHAPE";
        case GGML_OP_VIEW: return "VIEW";
        case GGML_OP_PERMUTE: return "PERMUTE";
        case GGML_OP_TRANSPOSE: return "TRANSPOSE";
        case GGML_OP_GLU: return "GLU";
        case GGML_OP_SUB: return "SUB";
        case GGML_OP_SCALE: return "SCALE";
        case GGML_OP_UNARY: return "UNARY";
        case GGML_OP_SQR: return "SQR";
        case GGML_OP_CPY: return "CPY";
        case GGML_OP_CONT: return "CONT";
        case GGML_OP_DUP: return "DUP";
        case GGML_OP_ROPE: return "ROPE";
        case GGML_OP_GET_ROWS: return "GET_ROWS";
        case GGML_OP_SET_ROWS: return "SET_ROWS";
        case GGML_OP_SOFT_MAX: return "SOFT_MAX";
        case GGML_OP_FLASH_ATTN_EXT: return "FLASH_ATTN_EXT";
        default: return "OP";
    }
}
const char* ggml_type_name(enum ggml_type t) {
    switch (t) {
        case GGML_TYPE_F32: return "f32";
        case GGML_TYPE_Q4_0: return "q4_0";
        case GGML_TYPE_Q8_0: return "q8_0";
        case GGML_TYPE_Q4_K: return "q4_K";
        case GGML_TYPE_Q6_K: return "q6_K";
        case GGML_TYPE_Q5_K: return "q5_K";
        case GGML_TYPE_IQ4_XS: return "iq4_xs";
        case GGML_TYPE_Q3_K: return "q3_K";
        case GGML_TYPE_Q2_K: return "q2_K";
        case GGML_TYPE_Q4_1: return "q4_1";
        case GGML_TYPE_Q5_1: return "q5_1";
        case GGML_TYPE_Q5_0: return "q5_0";
        case GGML_TYPE_IQ4_NL: return "iq4_nl";
        case GGML_TYPE_F16: return "f16";
        case GGML_TYPE_I32: return "i32";
        case GGML_TYPE_I64: return "i64";
        default: return "?";
    }
}
int ggml_graph_n_nodes(ggml_cgraph* g) { return g->n_nodes; }
ggml_tensor* ggml_graph_node(ggml_cgraph* g, int i) { return g->nodes[i < 0 ? g->n_nodes + i : i]; }
ggml_backend_buffer_t ggml_backend_buffer_init(ggml_backend_buffer_type_t buft, ggml_backend_buffer_i iface, void* context,
                                               size_t size) {
    ggml_backend_buffer* b = new ggml_backend_buffer();
    b->iface = iface;
    b->buft = buft;
    b->context = context;
    b->size = size;
    b->usage = GGML_BACKEND_BUFFER_USAGE_ANY;
    return b;
}
bool ggml_guid_matches(ggml_guid_t a, ggml_guid_t b) { return memcmp(a, b, sizeof(ggml_guid)) == 0; }
static ggml_backend_reg_t g_registered = nullptr;
void ggml_backend_register(ggml_backend_reg_t reg) { g_registered = reg; }
ggml_backend_dev_t ggml_backend_get_device(ggml_backend_t backend) { return backend->device; }
size_t ggml_backend_buffer_get_size(ggml_backend_buffer_t buffer) { return buffer->size; }
enum ggml_backend_buffer_usage ggml_backend_buffer_get_usage(ggml_backend_buffer_t buffer) { return buffer->usage; }
ggml_backend_buffer_type_t ggml_backend_buffer_get_type(ggml_backend_buffer_t buffer) { return buffer->buft; }
ggml_backend_dev_t ggml_backend_buft_get_device(ggml_backend_buffer_type_t buft) { return buft->device; }
ggml_backend_reg_t ggml_backend_dev_backend_reg(ggml_backend_dev_t device) { return device->reg; }
size_t ggml_tensor_overhead(void) { return sizeof(ggml_tensor) + 32; }
ggml_context* ggml_init(ggml_init_params) { return new ggml_context(); }
void ggml_free(ggml_context* ctx) {
    if (!ctx) return;
    for (ggml_tensor* t : ctx->tensors) delete t;
    delete ctx;
}
ggml_tensor* ggml_new_tensor_2d(ggml_context* ctx, enum ggml_type type, int64_t ne0, int64_t ne1) {
    ggml_tensor* t = new ggml_tensor();
    memset(t, 0, sizeof(*t));
    size_t ts;
    int64_t bs;
    traits(type, &ts, &bs);
    t->type = type;
    t->ne[0] = ne0; t->ne[1] = ne1; t->ne[2] = 1; t->ne[3] = 1;
    t->nb[0] = ts; t->nb[1] = ts * (size_t)(ne0 / bs); t->nb[2] = t->nb[1] * (size_t)ne1; t->nb[3] = t->nb[2];
    ctx->tensors.push_back(t);
    return t;
}
ggml_tensor* ggml_mul_mat(ggml_context* ctx, ggml_tensor* a, ggml_tensor* b) {
    ggml_tensor* c = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, a->ne[1], b->ne[1]);
    c->op = GGML_OP_MUL_MAT;
    c->src[0] = a;
    c->src[1] = b;
    return c;
}
ggml_tensor* ggml_set_name(ggml_tensor* t, const char* name) {
    strncpy(t->name, name, sizeof(t->name) - 1);
    t->name[sizeof(t->name) - 1] = 0;
    return t;
}
const char* ggml_get_name(const ggml_tensor* t) { return t->name; }
}

#define CHECK(c)                                                                   \
    do {                                                                           \
        if (!(c)) {                                                                \
            fprintf(stderr, "driver: check failed at line %d: %s\n", __LINE__, #c); \
            return 1;                                                              \
        }                                                                          \
    } while (0)

static void shape(ggml_tensor* t, enum ggml_type type, int64_t ne0, int64_t ne1, const char* name) {
    memset(t, 0, sizeof(*t));
    size_t ts;
    int64_t bs;
    traits(type, &ts, &bs);
    t->type = type;
    t->ne[0] = ne0; t->ne[1] = ne1; t->ne[2] = 1; t->ne[3] = 1;
    t->nb[0] = ts; t->nb[1] = ts * (size_t)(ne0 / bs); t->nb[2] = t->nb[1] * (size_t)ne1; t->nb[3] = t->nb[2];
    t->op = GGML_OP_NONE;
    snprintf(t->name, sizeof(t->name), "%s", name);
}

static std::vector<uint8_t> slurp(const std::string& path) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) { perror(path.c_str()); exit(2); }
    fseek(f, 0, SEEK_END);
    long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    std::vector<uint8_t> v((size_t)n);
    if (fread(v.data(), 1, v.size(), f) != v.size()) exit(2);
    fclose(f);
    return v;
}
static bool dump(const std::string& path, const void* p, size_t n) {
    FILE* f = fopen(path.c_str(), "wb");
    if (!f) return false;
    const bool ok = fwrite(p, 1, n, f) == n;
    fclose(f);
    return ok;
}

// what ggml's allocator does: every tensor padded to the buffer type's alignment, one buffer
struct Arena {
    ggml_backend_buffer_type_t buft;
    std::vector<ggml_tensor*> tensors;
    std::vector<size_t> offsets;
    size_t total = 0;
    ggml_backend_buffer_t buf = nullptr;
    bool weights = true;   // the usage llama.cpp gives the buffers it loads the model into; false: a compute / cache buffer
    void add(ggml_tensor* t) {
        tensors.push_back(t);
        offsets.push_back(total);
        total += (buft->iface.get_alloc_size(buft, t) + 63) & ~(size_t)63;
    }
    bool commit() {
        buf = buft->iface.alloc_buffer(buft, total);
        if (!buf) return false;
        buf->usage = weights ? GGML_BACKEND_BUFFER_USAGE_WEIGHTS : GGML_BACKEND_BUFFER_USAGE_ANY;
        char* base = (char*)buf->iface.get_base(buf);
        for (size_t i = 0; i < tensors.size(); ++i) {
            tensors[i]->buffer = buf;
            tensors[i]->data = base + offsets[i];
        }
        buf->iface.clear(buf, 0);
        return true;
    }
};

static int run_mulmat(int argc, char** argv, ggml_backend_dev_t dev, ggml_backend_buffer_type_t buft) {
    CHECK(argc == 9);
    const enum ggml_type type = (enum ggml_type)atoi(argv[2]);
    const int64_t M = atoll(argv[3]), N = atoll(argv[4]), K = atoll(argv[5]);
    std::vector<uint8_t> wbytes = slurp(argv[6]), xbytes = slurp(argv[7]);

    ggml_backend_dev_props props;
    dev->iface.get_props(dev, &props);
    CHECK(!props.caps.async && !props.caps.host_buffer && !props.caps.events);
    printf("device: %s\n", props.description);
    ggml_backend_t backend = dev->iface.init_backend(dev, nullptr);
    CHECK(backend && backend->iface.graph_compute && backend->iface.synchronize == nullptr);
    CHECK(ggml_backend_is_ameva(backend));

    ggml_tensor w, x, y, bad;
    shape(&w, type, K, N, "weight");
    shape(&x, GGML_TYPE_F32, K, M, "activations");
    shape(&y, GGML_TYPE_F32, N, M, "result");
    shape(&bad, GGML_TYPE_F32, N, M, "difference");
    CHECK(wbytes.size() == ggml_nbytes(&w) && xbytes.size() == ggml_nbytes(&x));
    CHECK(buft->iface.get_alloc_size(buft, &w) >= ggml_nbytes(&w));
    CHECK(buft->iface.get_alloc_size(buft, &x) == ggml_nbytes(&x));
    Arena ar{buft};
    ar.add(&w);
    ar.add(&x);
    ar.add(&y);
    CHECK(ar.commit());
    ggml_backend_buffer_t buf = ar.buf;
    buf->iface.set_tensor(buf, &w, wbytes.data(), 0, wbytes.size());
    buf->iface.set_tensor(buf, &x, xbytes.data(), 0, xbytes.size());

    // read-back: whole tensor and an odd partial range return the uploaded ggml bytes
    std::vector<uint8_t> back(wbytes.size());
    buf->iface.get_tensor(buf, &w, back.data(), 0, back.size());
    CHECK(back == wbytes);
    const size_t po = wbytes.size() / 3 + 1, pn = wbytes.size() / 5 + 3;
    std::vector<uint8_t> part(pn);
    buf->iface.get_tensor(buf, &w, part.data(), po, pn);
    CHECK(memcmp(part.data(), wbytes.data() + po, pn) == 0);
    // a partial upload patches exactly its range
    std::vector<uint8_t> scrambled = wbytes;
    for (size_t i = po; i < po + pn; ++i) scrambled[i] ^= 0x5A;
    buf->iface.set_tensor(buf, &w, scrambled.data() + po, po, pn);
    buf->iface.get_tensor(buf, &w, back.data(), 0, back.size());
    CHECK(back == scrambled);
    buf->iface.set_tensor(buf, &w, wbytes.data() + po, po, pn);   // and back

    y.op = GGML_OP_MUL_MAT;
    y.src[0] = &w;
    y.src[1] = &x;
    CHECK(dev->iface.supports_op(dev, &y));
    ggml_tensor* nodes[2] = {&y, &bad};
    ggml_cgraph graph = {1, nodes};
    CHECK(backend->iface.graph_compute(backend, &graph) == GGML_STATUS_SUCCESS);
    std::vector<uint8_t> out(ggml_nbytes(&y));
    buf->iface.get_tensor(buf, &y, out.data(), 0, out.size());
    CHECK(dump(argv[8], out.data(), out.size()));

    // a graph with a node this backend cannot run is refused as a whole: the result buffer stays untouched
    bad.op = GGML_OP_SUB;
    bad.src[0] = &y;
    bad.src[1] = &y;
    bad.buffer = buf;
    bad.data = y.data;
    CHECK(!dev->iface.supports_op(dev, &bad));
    buf->iface.memset_tensor(buf, &y, 0xEE, 0, ggml_nbytes(&y));
    graph.n_nodes = 2;
    const int64_t ops_before = ggml_backend_ameva_get_gpu_op_count();
    CHECK(backend->iface.graph_compute(backend, &graph) == GGML_STATUS_FAILED);
    CHECK(ggml_backend_ameva_get_gpu_op_count() == ops_before);
    std::vector<uint8_t> after(ggml_nbytes(&y));
    buf->iface.get_tensor(buf, &y, after.data(), 0, after.size());
    for (uint8_t v : after) CHECK(v == 0xEE);

    buf->iface.free_buffer(buf);
    delete buf;
    backend->iface.free(backend);
    ggml_backend_ameva_teardown();
    CHECK(ggml_backend_ameva_get_context_destroy_count() == ggml_backend_ameva_get_context_create_count());
    printf("ok\n");
    return 0;
}

static ggml_tensor* op2(ggml_tensor* t, enum ggml_op op, ggml_tensor* a, ggml_tensor* b) {
    t->op = op;
    t->src[0] = a;
    t->src[1] = b;
    return t;
}

static int run_layer(int argc, char** argv, ggml_backend_dev_t dev, ggml_backend_buffer_type_t buft) {
    CHECK(argc == 9);
    const enum ggml_type type = (enum ggml_type)atoi(argv[2]);
    const int64_t K = atoll(argv[3]), Nq = atoll(argv[4]), Nkv = atoll(argv[5]), Nff = atoll(argv[6]), M2 = atoll(argv[7]);
    const std::string dir = argv[8];
    auto in = [&](const char* n) { return slurp(dir + "/" + n); };
    auto out = [&](ggml_backend_buffer_t buf, ggml_tensor* t, const char* n) {
        std::vector<uint8_t> v(ggml_nbytes(t));
        buf->iface.get_tensor(buf, t, v.data(), 0, v.size());
        return dump(dir + "/" + n, v.data(), v.size());
    };
    ggml_backend_t backend = ggml_backend_ameva_init(0);
    CHECK(backend && ggml_backend_is_ameva(backend));
    CHECK(ggml_backend_ameva_init(1) == nullptr);
    CHECK(ggml_backend_ameva_buffer_type(0) == buft && ggml_backend_ameva_reg() == dev->reg);

    // weights: q (Nq rows), k, v (Nkv rows), o (K rows), gate / up (Nff rows), all over K; activations x (1 x K), a second
    // activation row `res` (K), the RMS weight row (K), x2 (M2 x K)
    ggml_tensor wq, wk, wv, wo, wg, wu, x, res, rw, x2;
    shape(&wq, type, K, Nq, "wq");
    shape(&wk, type, K, Nkv, "wk");
    shape(&wv, type, K, Nkv, "wv");
    shape(&wo, type, K, K, "wo");
    shape(&wg, type, K, Nff, "w_gate");
    shape(&wu, type, K, Nff, "w_up");
    shape(&x, GGML_TYPE_F32, K, 1, "x");
    shape(&res, GGML_TYPE_F32, K, 1, "residual");
    shape(&rw, GGML_TYPE_F32, K, 1, "rms_weight");
    shape(&x2, GGML_TYPE_F32, K, M2, "x2");
    // results
    ggml_tensor rn, xn, q, k, v, o, o_res, gate, up, act, wq_rows, qv, y2;
    shape(&rn, GGML_TYPE_F32, K, 1, "rms_norm");
    shape(&xn, GGML_TYPE_F32, K, 1, "x_normed");
    shape(&q, GGML_TYPE_F32, Nq, 1, "q");
    shape(&k, GGML_TYPE_F32, Nkv, 1, "k");
    shape(&v, GGML_TYPE_F32, Nkv, 1, "v");
    shape(&o, GGML_TYPE_F32, K, 1, "o");
    shape(&o_res, GGML_TYPE_F32, K, 1, "o_plus_residual");
    shape(&gate, GGML_TYPE_F32, Nff, 1, "gate");
    shape(&up, GGML_TYPE_F32, Nff, 1, "up");
    shape(&act, GGML_TYPE_F32, Nff, 1, "swiglu");
    // rows [Nq / 2, Nq) of wq, as a view (what ggml_view_2d makes): same K, same row pitch, data = base + offset
    shape(&wq_rows, type, K, Nq - Nq / 2, "wq_rows");
    shape(&qv, GGML_TYPE_F32, Nq - Nq / 2, 1, "q_of_row_range");
    shape(&y2, GGML_TYPE_F32, Nq, M2, "y2");

    Arena ar{buft};
    for (ggml_tensor* t : {&wq, &wk, &wv, &wo, &wg, &wu, &x, &res, &rw, &x2, &rn, &xn, &q, &k, &v, &o, &o_res, &gate, &up, &act, &qv, &y2})
        ar.add(t);
    CHECK(ar.commit());
    ggml_backend_buffer_t buf = ar.buf;
    wq_rows.view_src = &wq;
    wq_rows.view_offs = (size_t)(Nq / 2) * wq.nb[1];
    wq_rows.buffer = buf;
    wq_rows.data = (char*)wq.data + wq_rows.view_offs;
    wq_rows.op = GGML_OP_VIEW;
    wq_rows.src[0] = &wq;

    const int64_t repacked_before = ggml_backend_ameva_get_repacked_tensor_count();
    struct { ggml_tensor* t; const char* file; } uploads[] = {{&wq, "wq.bin"}, {&wk, "wk.bin"}, {&wv, "wv.bin"}, {&wo, "wo.bin"},
                                                              {&wg, "wg.bin"}, {&wu, "wu.bin"}, {&x, "x.bin"},   {&res, "res.bin"},
                                                              {&rw, "rw.bin"}, {&x2, "x2.bin"}};
    for (auto& u : uploads) {
        std::vector<uint8_t> bytes = in(u.file);
        CHECK(bytes.size() == ggml_nbytes(u.t));
        buf->iface.set_tensor(buf, u.t, bytes.data(), 0, bytes.size());
    }
    CHECK(ggml_backend_ameva_get_repacked_tensor_count() == repacked_before + 6);
    CHECK(ggml_backend_ameva_get_repacked_bytes() > 0);
    // the view reads back the bytes of its rows
    {
        std::vector<uint8_t> all = in("wq.bin"), part(ggml_nbytes(&wq_rows));
        buf->iface.get_tensor(buf, &wq_rows, part.data(), 0, part.size());
        CHECK(memcmp(part.data(), all.data() + wq_rows.view_offs, part.size()) == 0);
    }

    // ---- graph 1: one activation row through a decoder-layer-shaped graph ----
    op2(&rn, GGML_OP_RMS_NORM, &x, nullptr);
    const float eps = 1e-5f;
    memcpy(&rn.op_params[0], &eps, 4);
    op2(&xn, GGML_OP_MUL, &rn, &rw);
    op2(&q, GGML_OP_MUL_MAT, &wq, &xn);
    op2(&k, GGML_OP_MUL_MAT, &wk, &xn);
    op2(&v, GGML_OP_MUL_MAT, &wv, &xn);
    op2(&o, GGML_OP_MUL_MAT, &wo, &res);   // another activation row: not part of the q / k / v group
    op2(&o_res, GGML_OP_ADD, &o, &x);      // its consumer: computed by the same launch
    op2(&gate, GGML_OP_MUL_MAT, &wg, &xn);
    op2(&up, GGML_OP_MUL_MAT, &wu, &xn);
    op2(&act, GGML_OP_GLU, &gate, &up);
    act.op_params[0] = (int32_t)GGML_GLU_OP_SWIGLU;
    act.op_params[1] = 0;
    op2(&qv, GGML_OP_MUL_MAT, &wq_rows, &xn);
    ggml_tensor* nodes1[] = {&rn, &xn, &q, &k, &v, &o, &o_res, &gate, &up, &act, &wq_rows, &qv};
    const int n1 = (int)(sizeof(nodes1) / sizeof(nodes1[0]));
    for (ggml_tensor* t : nodes1) CHECK(dev->iface.supports_op(dev, t));
    ggml_cgraph g1 = {n1, nodes1};
    ggml_backend_ameva_reset_counters();
    CHECK(backend->iface.graph_compute(backend, &g1) == GGML_STATUS_SUCCESS);
    printf("COUNTER gpu_op %lld\n", (long long)ggml_backend_ameva_get_gpu_op_count());
    printf("COUNTER mul_mat %lld\n", (long long)ggml_backend_ameva_get_f32_gpu_sgemm_dispatch_count());
    printf("COUNTER fused_pair %lld\n", (long long)ggml_backend_ameva_get_fused_pair_count());
    printf("COUNTER qmv %lld\n", (long long)ggml_backend_ameva_get_qmv_mul_mat_count());
    printf("COUNTER mmq %lld\n", (long long)ggml_backend_ameva_get_mmq_mul_mat_count());
    printf("COUNTER mmqb %lld\n", (long long)ggml_backend_ameva_get_mmqb_mul_mat_count());
    CHECK(ggml_backend_ameva_get_gpu_op_count() == 11);   // every node but the view
    CHECK(ggml_backend_ameva_get_f32_gpu_sgemm_dispatch_count() == 7 && ggml_backend_ameva_get_qmv_mul_mat_count() == 7);
    CHECK(ggml_backend_ameva_get_q5_0_cpu_dequant_count() == 0);
    CHECK(out(buf, &xn, "xn.out") && out(buf, &q, "q.out") && out(buf, &k, "k.out") && out(buf, &v, "v.out") &&
          out(buf, &o_res, "o_res.out") && out(buf, &act, "act.out") && out(buf, &qv, "qv.out") && out(buf, &gate, "gate.out"));

    // ---- graph 2: more activation rows than graph 1 reserved scratch for, and two nodes sharing src1 ----
    ggml_tensor y2b;
    shape(&y2b, GGML_TYPE_F32, Nq, M2, "y2_again");
    y2b.buffer = buf;
    y2b.data = y2.data;   // the second product overwrites the first: same src1, quantized once
    op2(&y2, GGML_OP_MUL_MAT, &wq, &x2);
    op2(&y2b, GGML_OP_MUL_MAT, &wq, &x2);
    ggml_tensor* nodes2[] = {&y2, &y2b};
    ggml_cgraph g2 = {2, nodes2};
    CHECK(backend->iface.graph_compute(backend, &g2) == GGML_STATUS_SUCCESS);
    CHECK(ggml_backend_ameva_get_gpu_op_count() == 13);
    CHECK(out(buf, &y2, "y2.out"));
    // and graph 1 again after the scratch grew
    CHECK(backend->iface.graph_compute(backend, &g1) == GGML_STATUS_SUCCESS);
    CHECK(out(buf, &q, "q_again.out"));

    // ---- host-side failure injection: FAILED, and the op counter does not move (tests/test_amuda_ggml_backend.cpp:211-251) ----
    int gates = 0;
    for (int point = AMEVA_FAIL_MAP_SRC0; point <= AMEVA_FAIL_TENSOR_RANGE_OOB; ++point) {
        const int64_t before = ggml_backend_ameva_get_gpu_op_count();
        ggml_backend_ameva_set_failure_injection((AmevaFailureInjectionPoint)point);
        CHECK(ggml_backend_ameva_get_failure_injection() == (AmevaFailureInjectionPoint)point);
        const enum ggml_status st = backend->iface.graph_compute(backend, &g1);
        const bool ok = st == GGML_STATUS_FAILED && ggml_backend_ameva_get_gpu_op_count() == before;
        printf("GATE_%02d: %s\n", point, ok ? "PASS" : "FAIL");
        gates += ok;
    }
    ggml_backend_ameva_set_failure_injection(AMEVA_FAIL_NONE);
    printf("FAILURE_GATES=%d/10\n", gates);
    CHECK(gates == 10);
    CHECK(backend->iface.graph_compute(backend, &g1) == GGML_STATUS_SUCCESS);   // and the backend still works

    // ---- registration and teardown ----
    ggml_backend_ameva_register();
    CHECK(g_registered == dev->reg);
    CHECK(dev->reg->iface.get_proc_address(dev->reg, "ggml_backend_ameva_get_gpu_op_count") == (void*)ggml_backend_ameva_get_gpu_op_count);
    CHECK(dev->reg->iface.get_proc_address(dev->reg, "no_such_function") == nullptr);
    ggml_backend_ameva_teardown();   // refused while a backend and a buffer are alive
    CHECK(ggml_backend_ameva_get_context_destroy_count() == 0);
    buf->iface.free_buffer(buf);
    delete buf;
    backend->iface.free(backend);
    ggml_backend_ameva_teardown();
    CHECK(ggml_backend_ameva_get_context_destroy_count() == 1 && ggml_backend_ameva_get_context_create_count() == 1);
    CHECK(ggml_backend_ameva_get_kernel_create_count() == ggml_backend_ameva_get_kernel_destroy_count());
    printf("ok\n");
    return 0;
}

// a contiguous tensor of up to three dimensions
static void shape3(ggml_tensor* t, enum ggml_type type, int64_t ne0, int64_t ne1, int64_t ne2, const char* name) {
    shape(t, type, ne0, ne1, name);
    t->ne[2] = ne2;
    t->nb[3] = t->nb[2] * (size_t)ne2;
}
// a strided view of `base` starting `offs` bytes in
static void view3(ggml_tensor* t, ggml_tensor* base, int64_t ne0, int64_t ne1, int64_t ne2, size_t nb1, size_t nb2, size_t offs,
                  enum ggml_op op, const char* name) {
    shape3(t, base->type, ne0, ne1, ne2, name);
    t->nb[1] = nb1;
    t->nb[2] = nb2;
    t->nb[3] = nb2 * (size_t)ne2;
    t->view_src = base;
    t->view_offs = offs;
    t->buffer = base->buffer;
    t->data = (char*)base->data + offs;
    t->op = op;
    t->src[0] = base;
}

// A quantized KV cache (q8_0 / q4_0 tensors in a buffer whose usage is not WEIGHTS keep ggml's block layout):
// kvq <type> <D> <n_head> <n_head_kv> <n_ctx> <n_kv> <n_tok> <dir>. SET_ROWS of the new keys / values into the caches,
// FLASH_ATTN_EXT over strided views of them, CPY of the key view to f32 and CPY of the new keys to a quantized tensor of
// the same shape. Reads q.bin, kcur.bin, vcur.bin, kcache.bin, vcache.bin (ggml blocks), slots.bin, mask.bin; writes
// attn.out, kcache.out, vcache.out (ggml blocks), kdeq.out, kcur_q.out.
static int run_kvq(int argc, char** argv, ggml_backend_dev_t dev, ggml_backend_buffer_type_t buft) {
    CHECK(argc == 10);
    const enum ggml_type type = (enum ggml_type)atoi(argv[2]);
    const int64_t D = atoll(argv[3]), n_head = atoll(argv[4]), n_head_kv = atoll(argv[5]), n_ctx = atoll(argv[6]),
                  n_kv = atoll(argv[7]), n_tok = atoll(argv[8]);
    const std::string dir = argv[9];
    auto in = [&](const char* n) { return slurp(dir + "/" + n); };
    ggml_backend_t backend = dev->iface.init_backend(dev, nullptr);
    CHECK(backend);
    const int64_t kvw = D * n_head_kv;
    ggml_tensor q, kcur, vcur, kcache, vcache, slots, mask, attn, kdeq, kcur_q;
    shape3(&q, GGML_TYPE_F32, D, n_tok, n_head, "q");
    shape(&kcur, GGML_TYPE_F32, kvw, n_tok, "k_cur");
    shape(&vcur, GGML_TYPE_F32, kvw, n_tok, "v_cur");
    shape(&kcache, type, kvw, n_ctx, "cache_k");
    shape(&vcache, type, kvw, n_ctx, "cache_v");
    shape(&slots, GGML_TYPE_I64, n_tok, 1, "slots");
    shape(&mask, GGML_TYPE_F16, n_kv, n_tok, "kq_mask");
    shape3(&attn, GGML_TYPE_F32, D, n_head, n_tok, "kqv");
    shape3(&kdeq, GGML_TYPE_F32, D, n_kv, n_head_kv, "k_f32");
    shape(&kcur_q, type, kvw, n_tok, "k_cur_q");
    Arena ar{buft};
    ar.weights = false;   // a cache / compute buffer: quantized tensors stay in ggml's layout
    for (ggml_tensor* t : {&q, &kcur, &vcur, &kcache, &vcache, &slots, &mask, &attn, &kdeq, &kcur_q}) ar.add(t);
    CHECK(ar.commit());
    ggml_backend_buffer_t buf = ar.buf;
    struct { ggml_tensor* t; const char* file; } uploads[] = {{&q, "q.bin"}, {&kcur, "kcur.bin"}, {&vcur, "vcur.bin"},
        {&kcache, "kcache.bin"}, {&vcache, "vcache.bin"}, {&slots, "slots.bin"}, {&mask, "mask.bin"}};
    for (auto& u : uploads) {
        std::vector<uint8_t> bytes = in(u.file);
        CHECK(bytes.size() == ggml_nbytes(u.t));
        buf->iface.set_tensor(buf, u.t, bytes.data(), 0, bytes.size());
    }
    {   // the cache is not repacked: its bytes read back as they were written, also from an odd range
        std::vector<uint8_t> want = in("kcache.bin"), got(want.size());
        buf->iface.get_tensor(buf, &kcache, got.data(), 0, got.size());
        CHECK(got == want);
    }
    ggml_tensor kset, vset, k_view, v_view;
    view3(&kset, &kcache, kvw, n_ctx, 1, kcache.nb[1], kcache.nb[2], 0, GGML_OP_SET_ROWS, "cache_k_set");
    kset.src[0] = &kcur;
    kset.src[1] = &slots;
    view3(&vset, &vcache, kvw, n_ctx, 1, vcache.nb[1], vcache.nb[2], 0, GGML_OP_SET_ROWS, "cache_v_set");
    vset.src[0] = &vcur;
    vset.src[1] = &slots;
    const size_t head_bytes = (size_t)(D / 32) * kcache.nb[0];
    view3(&k_view, &kcache, D, n_kv, n_head_kv, kcache.nb[1], head_bytes, 0, GGML_OP_VIEW, "k_view");
    view3(&v_view, &vcache, D, n_kv, n_head_kv, vcache.nb[1], head_bytes, 0, GGML_OP_VIEW, "v_view");
    op2(&attn, GGML_OP_FLASH_ATTN_EXT, &q, &k_view);
    attn.src[2] = &v_view;
    attn.src[3] = &mask;
    const float scale = 1.0f / sqrtf((float)D), zero = 0.0f;
    memcpy(&attn.op_params[0], &scale, 4);
    memcpy(&attn.op_params[1], &zero, 4);
    memcpy(&attn.op_params[2], &zero, 4);
    op2(&kdeq, GGML_OP_CPY, &k_view, &kdeq);
    op2(&kcur_q, GGML_OP_CPY, &kcur, &kcur_q);
    ggml_tensor* nodes[] = {&kset, &vset, &k_view, &v_view, &attn, &kdeq, &kcur_q};
    const int n = (int)(sizeof(nodes) / sizeof(nodes[0]));
    for (ggml_tensor* t : nodes) CHECK(dev->iface.supports_op(dev, t));
    ggml_cgraph g = {n, nodes};
    CHECK(backend->iface.graph_compute(backend, &g) == GGML_STATUS_SUCCESS);
    auto out = [&](ggml_tensor* t, const char* name) {
        std::vector<uint8_t> v(ggml_nbytes(t));
        buf->iface.get_tensor(buf, t, v.data(), 0, v.size());
        return dump(dir + "/" + name, v.data(), v.size());
    };
    CHECK(out(&attn, "attn.out") && out(&kcache, "kcache.out") && out(&vcache, "vcache.out") && out(&kdeq, "kdeq.out") &&
          out(&kcur_q, "kcur_q.out"));
    buf->iface.free_buffer(buf);
    delete buf;
    backend->iface.free(backend);
    printf("ok\n");
    return 0;
}

// GET_ROWS from a quantized table uploaded like any weight (token embeddings): getrows <type> <rows> <nc> <n_idx> <dir>
// reads table.bin (ggml blocks) and idx.bin (i32), writes rows.bin (f32); an index outside the table must fail the graph.
static int run_getrows(int argc, char** argv, ggml_backend_dev_t dev, ggml_backend_buffer_type_t buft) {
    CHECK(argc == 7);
    const enum ggml_type type = (enum ggml_type)atoi(argv[2]);
    const int64_t rows = atoll(argv[3]), nc = atoll(argv[4]), n_idx = atoll(argv[5]);
    const std::string dir = argv[6];
    std::vector<uint8_t> tbytes = slurp(dir + "/table.bin"), ibytes = slurp(dir + "/idx.bin");
    ggml_backend_t backend = dev->iface.init_backend(dev, nullptr);
    CHECK(backend);
    ggml_tensor table, idx, out;
    shape(&table, type, nc, rows, "token_embd");
    shape(&idx, GGML_TYPE_I32, n_idx, 1, "tokens");
    shape(&out, GGML_TYPE_F32, nc, n_idx, "inp_embd");
    CHECK(tbytes.size() == ggml_nbytes(&table) && ibytes.size() == ggml_nbytes(&idx));
    Arena ar{buft};
    ar.add(&table);
    ar.add(&idx);
    ar.add(&out);
    CHECK(ar.commit());
    ggml_backend_buffer_t buf = ar.buf;
    buf->iface.set_tensor(buf, &table, tbytes.data(), 0, tbytes.size());
    buf->iface.set_tensor(buf, &idx, ibytes.data(), 0, ibytes.size());
    out.op = GGML_OP_GET_ROWS;
    out.src[0] = &table;
    out.src[1] = &idx;
    CHECK(dev->iface.supports_op(dev, &out));
    ggml_tensor* nodes[1] = {&out};
    ggml_cgraph graph = {1, nodes};
    CHECK(backend->iface.graph_compute(backend, &graph) == GGML_STATUS_SUCCESS);
    std::vector<uint8_t> res(ggml_nbytes(&out));
    buf->iface.get_tensor(buf, &out, res.data(), 0, res.size());
    CHECK(dump((dir + "/rows.bin").c_str(), res.data(), res.size()));
    int32_t bad = (int32_t)rows;
    buf->iface.set_tensor(buf, &idx, &bad, 4, 4);
    CHECK(backend->iface.graph_compute(backend, &graph) == GGML_STATUS_FAILED);
    buf->iface.free_buffer(buf);
    delete buf;
    backend->iface.free(backend);
    printf("ok\n");
    return 0;
}

// The ops around the mul_mats of a decoder layer, as llama.cpp strings them: token embedding (GET_ROWS), ROPE on the new
// queries and keys, the KV-cache write (SET_ROWS into f16 caches), attention of the new tokens over the cache
// (FLASH_ATTN_EXT on strided views of the caches) and a masked SOFT_MAX; then the same graph with a cache slot out of
// range, which must fail.
static int run_attn(int argc, char** argv, ggml_backend_dev_t dev, ggml_backend_buffer_type_t buft) {
    CHECK(argc == 11);
    const int64_t D = atoll(argv[2]), n_head = atoll(argv[3]), n_head_kv = atoll(argv[4]), n_ctx = atoll(argv[5]),
                  n_kv = atoll(argv[6]), n_tok = atoll(argv[7]), n_vocab = atoll(argv[8]), n_embd = atoll(argv[9]);
    const std::string dir = argv[10];
    auto in = [&](const char* n) { return slurp(dir + "/" + n); };
    ggml_backend_t backend = ggml_backend_ameva_init(0);
    CHECK(backend);
    const int64_t kvw = D * n_head_kv;   // floats of one cache row
    ggml_tensor emb, tok, q, kcur, vcur, kcache, vcache, pos, slots, mask, sc, smask;
    shape(&emb, GGML_TYPE_F16, n_embd, n_vocab, "token_embd");
    shape(&tok, GGML_TYPE_I32, n_tok, 1, "tokens");
    shape3(&q, GGML_TYPE_F32, D, n_head, n_tok, "q");
    shape3(&kcur, GGML_TYPE_F32, D, n_head_kv, n_tok, "k_cur");
    shape(&vcur, GGML_TYPE_F32, kvw, n_tok, "v_cur");
    shape(&kcache, GGML_TYPE_F16, kvw, n_ctx, "cache_k");
    shape(&vcache, GGML_TYPE_F16, kvw, n_ctx, "cache_v");
    shape(&pos, GGML_TYPE_I32, n_tok, 1, "pos");
    shape(&slots, GGML_TYPE_I64, n_tok, 1, "slots");
    shape(&mask, GGML_TYPE_F16, n_kv, n_tok, "kq_mask");
    shape3(&sc, GGML_TYPE_F32, n_kv, n_tok, n_head, "scores");
    shape(&smask, GGML_TYPE_F32, n_kv, n_tok, "scores_mask");
    ggml_tensor x, q_rope, k_rope, attn, sm;
    shape(&x, GGML_TYPE_F32, n_embd, n_tok, "inp_embd");
    shape3(&q_rope, GGML_TYPE_F32, D, n_head, n_tok, "q_rope");
    shape3(&k_rope, GGML_TYPE_F32, D, n_head_kv, n_tok, "k_rope");
    shape3(&attn, GGML_TYPE_F32, D, n_head, n_tok, "kqv");
    shape3(&sm, GGML_TYPE_F32, n_kv, n_tok, n_head, "soft_max");
    Arena ar{buft};
    for (ggml_tensor* t : {&emb, &tok, &q, &kcur, &vcur, &kcache, &vcache, &pos, &slots, &mask, &sc, &smask, &x, &q_rope, &k_rope,
                           &attn, &sm})
        ar.add(t);
    CHECK(ar.commit());
    ggml_backend_buffer_t buf = ar.buf;
    Arena ar2{buft};   // a second buffer of the same type, for the results of the copies below
    struct { ggml_tensor* t; const char* file; } uploads[] = {
        {&emb, "emb.bin"}, {&tok, "tok.bin"}, {&q, "q.bin"}, {&kcur, "kcur.bin"}, {&vcur, "vcur.bin"}, {&kcache, "kcache.bin"},
        {&vcache, "vcache.bin"}, {&pos, "pos.bin"}, {&slots, "slots.bin"}, {&mask, "mask.bin"}, {&sc, "sc.bin"}, {&smask, "smask.bin"}};
    for (auto& u : uploads) {
        std::vector<uint8_t> bytes = in(u.file);
        CHECK(bytes.size() == ggml_nbytes(u.t));
        buf->iface.set_tensor(buf, u.t, bytes.data(), 0, bytes.size());
    }
    // the graph
    op2(&x, GGML_OP_GET_ROWS, &emb, &tok);
    auto rope = [&](ggml_tensor* t, ggml_tensor* a) {
        op2(t, GGML_OP_ROPE, a, &pos);
        const float freq_base = 10000.0f, one = 1.0f, zero = 0.0f, bf = 32.0f, bs = 1.0f;
        t->op_params[1] = (int32_t)D;
        t->op_params[2] = 2;       // NEOX
        t->op_params[4] = 4096;
        memcpy(&t->op_params[5], &freq_base, 4);
        memcpy(&t->op_params[6], &one, 4);
        memcpy(&t->op_params[7], &zero, 4);
        memcpy(&t->op_params[8], &one, 4);
        memcpy(&t->op_params[9], &bf, 4);
        memcpy(&t->op_params[10], &bs, 4);
    };
    rope(&q_rope, &q);
    rope(&k_rope, &kcur);
    ggml_tensor k_rows, kset, vset, q_perm, k_view, v_view;
    view3(&k_rows, &k_rope, kvw, n_tok, 1, (size_t)kvw * 4, (size_t)kvw * n_tok * 4, 0, GGML_OP_RESHAPE, "k_rope_rows");
    // SET_ROWS: the node is a view of the cache it writes
    view3(&kset, &kcache, kvw, n_ctx, 1, kcache.nb[1], kcache.nb[2], 0, GGML_OP_SET_ROWS, "cache_k_set");
    kset.src[0] = &k_rows;
    kset.src[1] = &slots;
    view3(&vset, &vcache, kvw, n_ctx, 1, vcache.nb[1], vcache.nb[2], 0, GGML_OP_SET_ROWS, "cache_v_set");
    vset.src[0] = &vcur;
    vset.src[1] = &slots;
    // attention operands: q [D, n_tok, n_head] (a permutation of q_rope), the first n_kv rows of the caches by KV head
    view3(&q_perm, &q_rope, D, n_tok, n_head, (size_t)D * n_head * 4, (size_t)D * 4, 0, GGML_OP_PERMUTE, "q_perm");
    view3(&k_view, &kcache, D, n_kv, n_head_kv, kcache.nb[1], (size_t)D * 2, 0, GGML_OP_VIEW, "k_view");
    view3(&v_view, &vcache, D, n_kv, n_head_kv, vcache.nb[1], (size_t)D * 2, 0, GGML_OP_VIEW, "v_view");
    op2(&attn, GGML_OP_FLASH_ATTN_EXT, &q_perm, &k_view);
    attn.src[2] = &v_view;
    attn.src[3] = &mask;
    const float scale = 1.0f / sqrtf((float)D), zero = 0.0f;
    memcpy(&attn.op_params[0], &scale, 4);
    memcpy(&attn.op_params[1], &zero, 4);
    memcpy(&attn.op_params[2], &zero, 4);
    op2(&sm, GGML_OP_SOFT_MAX, &sc, &smask);
    memcpy(&sm.op_params[0], &scale, 4);
    memcpy(&sm.op_params[1], &zero, 4);
    // CONT of the permuted queries (a gather into [D, n_tok, n_head] order) and a CPY of the new values to f16
    ggml_tensor q_cont, v_f16;
    shape3(&q_cont, GGML_TYPE_F32, D, n_tok, n_head, "q_cont");
    shape(&v_f16, GGML_TYPE_F16, kvw, n_tok, "v_cur_f16");
    ar2.add(&q_cont);
    ar2.add(&v_f16);
    CHECK(ar2.commit());
    op2(&q_cont, GGML_OP_CONT, &q_perm, nullptr);
    op2(&v_f16, GGML_OP_CPY, &vcur, &v_f16);
    // SCALE with a bias, in place of nothing (own result), and SILU on the embedded rows
    ggml_tensor x_scaled, x_silu;
    shape(&x_scaled, GGML_TYPE_F32, n_embd, n_tok, "x_scaled");
    shape(&x_silu, GGML_TYPE_F32, n_embd, n_tok, "x_silu");
    Arena ar3{buft};
    ar3.add(&x_scaled);
    ar3.add(&x_silu);
    CHECK(ar3.commit());
    op2(&x_scaled, GGML_OP_SCALE, &x, nullptr);
    const float sc_s = 0.125f, sc_b = -0.5f;
    memcpy(&x_scaled.op_params[0], &sc_s, 4);
    memcpy(&x_scaled.op_params[1], &sc_b, 4);
    op2(&x_silu, GGML_OP_UNARY, &x, nullptr);
    x_silu.op_params[0] = (int32_t)GGML_UNARY_OP_SILU;
    ggml_tensor* nodes[] = {&x, &q_rope, &k_rope, &k_rows, &kset, &vset, &q_perm, &k_view, &v_view, &attn, &sm, &q_cont, &v_f16,
                            &x_scaled, &x_silu};
    const int n = (int)(sizeof(nodes) / sizeof(nodes[0]));
    for (ggml_tensor* t : nodes) CHECK(dev->iface.supports_op(dev, t));
    ggml_cgraph g = {n, nodes};
    ggml_backend_ameva_reset_counters();
    CHECK(backend->iface.graph_compute(backend, &g) == GGML_STATUS_SUCCESS);
    printf("COUNTER gpu_op %lld\n", (long long)ggml_backend_ameva_get_gpu_op_count());
    auto out = [&](ggml_tensor* t, const char* name) {
        std::vector<uint8_t> v(ggml_nbytes(t));
        buf->iface.get_tensor(buf, t, v.data(), 0, v.size());
        return dump(dir + "/" + name, v.data(), v.size());
    };
    {
        std::vector<uint8_t> v1(ggml_nbytes(&q_cont)), v2(ggml_nbytes(&v_f16));
        ar2.buf->iface.get_tensor(ar2.buf, &q_cont, v1.data(), 0, v1.size());
        ar2.buf->iface.get_tensor(ar2.buf, &v_f16, v2.data(), 0, v2.size());
        CHECK(dump(dir + "/q_cont.out", v1.data(), v1.size()) && dump(dir + "/v_f16.out", v2.data(), v2.size()));
        std::vector<uint8_t> v3(ggml_nbytes(&x_scaled)), v4(ggml_nbytes(&x_silu));
        ar3.buf->iface.get_tensor(ar3.buf, &x_scaled, v3.data(), 0, v3.size());
        ar3.buf->iface.get_tensor(ar3.buf, &x_silu, v4.data(), 0, v4.size());
        CHECK(dump(dir + "/x_scaled.out", v3.data(), v3.size()) && dump(dir + "/x_silu.out", v4.data(), v4.size()));
    }
    {   // a unary op the kernel has no code for is refused at planning time
        ggml_tensor t = x_silu;
        t.op_params[0] = (int32_t)GGML_UNARY_OP_ELU;
        CHECK(!dev->iface.supports_op(dev, &t));
    }
    CHECK(out(&x, "x.out") && out(&q_rope, "q_rope.out") && out(&k_rope, "k_rope.out") && out(&kcache, "kcache.out") &&
          out(&vcache, "vcache.out") && out(&attn, "attn.out") && out(&sm, "sm.out"));
    // a cache slot past the cache: the graph fails and the op counter does not move
    {
        std::vector<uint8_t> bytes = in("slots.bin");
        int64_t bad = n_ctx;
        memcpy(bytes.data(), &bad, 8);
        buf->iface.set_tensor(buf, &slots, bytes.data(), 0, bytes.size());
        const int64_t before = ggml_backend_ameva_get_gpu_op_count();
        CHECK(backend->iface.graph_compute(backend, &g) == GGML_STATUS_FAILED);
        CHECK(ggml_backend_ameva_get_gpu_op_count() == before);
    }
    // an op outside the set is refused at planning time
    sm.op_params[1] = 0x41000000;   // max_bias 8.0: ALiBi
    CHECK(!dev->iface.supports_op(dev, &sm));
    ar3.buf->iface.free_buffer(ar3.buf);
    ar2.buf->iface.free_buffer(ar2.buf);
    buf->iface.free_buffer(buf);
    backend->iface.free(backend);
    ggml_backend_ameva_teardown();
    printf("ok\n");
    return 0;
}

int main(int argc, char** argv) {
    CHECK(argc >= 2);
    CHECK(ggml_backend_ameva_abi_check() == nullptr);
    ggml_backend_reg_t reg = ggml_backend_init();
    CHECK(reg != nullptr);
    CHECK(reg->api_version == GGML_BACKEND_API_VERSION);
    CHECK(ggml_backend_score() == 100);
    CHECK(reg->iface.get_device_count(reg) == 1);
    ggml_backend_dev_t dev = reg->iface.get_device(reg, 0);
    CHECK(dev && dev->reg == reg && reg->iface.get_device(reg, 1) == nullptr);
    ggml_backend_buffer_type_t buft = dev->iface.get_buffer_type(dev);
    CHECK(buft && buft->device == dev);
    CHECK(buft->iface.get_alignment(buft) == 64);
    CHECK(!buft->iface.is_host(buft));
    CHECK(dev->iface.supports_buft(dev, buft));
    ggml_backend_buffer_type other{};
    CHECK(!dev->iface.supports_buft(dev, &other));
    CHECK(dev->iface.get_type(dev) == GGML_BACKEND_DEVICE_TYPE_GPU);
    printf("registry %s device %s buffer-type %s\n", reg->iface.get_name(reg), dev->iface.get_name(dev),
           buft->iface.get_name(buft));
    if (std::string(argv[1]) == "probe") {
        // what the scheduler asks at planning time, without a device: types and shapes only
        ggml_tensor w, x, y, a, b, c;
        shape(&w, GGML_TYPE_Q4_K, 512, 64, "w");
        shape(&x, GGML_TYPE_F32, 512, 3, "x");
        shape(&y, GGML_TYPE_F32, 64, 3, "y");
        op2(&y, GGML_OP_MUL_MAT, &w, &x);
        CHECK(dev->iface.supports_op(dev, &y));
        shape(&a, GGML_TYPE_F32, 64, 3, "a");
        shape(&b, GGML_TYPE_F32, 64, 1, "b");
        shape(&c, GGML_TYPE_F32, 64, 3, "c");
        op2(&c, GGML_OP_ADD, &a, &b);
        CHECK(dev->iface.supports_op(dev, &c));
        c.op = GGML_OP_SUB;
        CHECK(!dev->iface.supports_op(dev, &c));
        CHECK(ggml_backend_ameva_get_supports_query_count() == 3 && ggml_backend_ameva_get_supported_op_count() == 2);
        CHECK(ggml_backend_ameva_get_context_create_count() == 0);   // nothing above touched the device
        printf("build %s\n", ggml_backend_ameva_get_build_commit());
        return 0;
    }
    if (std::string(argv[1]) == "mulmat") return run_mulmat(argc, argv, dev, buft);
    if (std::string(argv[1]) == "layer") return run_layer(argc, argv, dev, buft);
    if (std::string(argv[1]) == "attn") return run_attn(argc, argv, dev, buft);
    if (std::string(argv[1]) == "getrows") return run_getrows(argc, argv, dev, buft);
    if (std::string(argv[1]) == "kvq") return run_kvq(argc, argv, dev, buft);
    fprintf(stderr, "driver: unknown mode %s\n", argv[1]);
    return 2;
}
