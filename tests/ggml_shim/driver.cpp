// Test harness for the ggml backend plugin (libggml-ameva-b200.so). It stands in for the host application: a minimal
// ggml-base (the six functions the plugin calls, restated for the four tensor types of the test) and a driver that walks
// the plugin's tables the way ggml's loader, allocator and scheduler do. Built against the host's ggml headers; not part
// of the product.
//
//   driver probe                                   registry / device / buffer-type facts, no device needed
//   driver mulmat <type> <M> <N> <K> <w.bin> <x.bin> <y.bin>
//                                                  uploads ggml blocks + f32 activations, runs a one-node MUL_MAT graph,
//                                                  writes y; also checks weight read-back (whole, partial), a partial
//                                                  set_tensor, and that a graph with an unsupported node is refused
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "ggml-backend-impl.h"
#include "ggml-backend.h"
#include "ggml.h"

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
        default: fprintf(stderr, "shim: type %d not in the test set\n", (int)t); abort();
    }
}

extern "C" {
size_t ggml_nbytes(const ggml_tensor* t) {
    size_t ts;
    int64_t bs;
    traits(t->type, &ts, &bs);
    return (size_t)(t->ne[0] / bs) * ts * (size_t)(t->ne[1] * t->ne[2] * t->ne[3]);
}
bool ggml_is_contiguous(const ggml_tensor* t) {
    size_t ts;
    int64_t bs;
    traits(t->type, &ts, &bs);
    return t->nb[0] == ts && t->nb[1] == ts * (size_t)(t->ne[0] / bs) && t->nb[2] == t->nb[1] * (size_t)t->ne[1] &&
           t->nb[3] == t->nb[2] * (size_t)t->ne[2];
}
const char* ggml_op_name(enum ggml_op op) { return op == GGML_OP_MUL_MAT ? "MUL_MAT" : (op == GGML_OP_ADD ? "ADD" : "OP"); }
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
ggml_backend_reg_t ggml_backend_init(void);
int ggml_backend_score(void);
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

static std::vector<uint8_t> slurp(const char* path) {
    FILE* f = fopen(path, "rb");
    if (!f) { perror(path); exit(2); }
    fseek(f, 0, SEEK_END);
    long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    std::vector<uint8_t> v((size_t)n);
    if (fread(v.data(), 1, v.size(), f) != v.size()) exit(2);
    fclose(f);
    return v;
}

int main(int argc, char** argv) {
    CHECK(argc >= 2);
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
    if (std::string(argv[1]) == "probe") return 0;

    CHECK(std::string(argv[1]) == "mulmat" && argc == 9);
    const enum ggml_type type = (enum ggml_type)atoi(argv[2]);
    const int64_t M = atoll(argv[3]), N = atoll(argv[4]), K = atoll(argv[5]);
    std::vector<uint8_t> wbytes = slurp(argv[6]), xbytes = slurp(argv[7]);

    ggml_backend_dev_props props;
    dev->iface.get_props(dev, &props);
    CHECK(!props.caps.async && !props.caps.host_buffer && !props.caps.events);
    printf("device: %s\n", props.description);
    ggml_backend_t backend = dev->iface.init_backend(dev, nullptr);
    CHECK(backend && backend->iface.graph_compute && backend->iface.synchronize == nullptr);

    ggml_tensor w, x, y, bad;
    shape(&w, type, K, N, "weight");
    shape(&x, GGML_TYPE_F32, K, M, "activations");
    shape(&y, GGML_TYPE_F32, N, M, "result");
    shape(&bad, GGML_TYPE_F32, N, M, "sum");
    CHECK(wbytes.size() == ggml_nbytes(&w) && xbytes.size() == ggml_nbytes(&x));
    CHECK(buft->iface.get_alloc_size(buft, &w) >= ggml_nbytes(&w));
    CHECK(buft->iface.get_alloc_size(buft, &x) == ggml_nbytes(&x));
    // what ggml's allocator does: pad every tensor to the alignment, one buffer
    auto pad = [](size_t v) { return (v + 63) & ~(size_t)63; };
    const size_t ow = 0, ox = ow + pad(buft->iface.get_alloc_size(buft, &w)), oy = ox + pad(ggml_nbytes(&x)),
                 total = oy + pad(ggml_nbytes(&y));
    ggml_backend_buffer_t buf = buft->iface.alloc_buffer(buft, total);
    CHECK(buf != nullptr);
    char* base = (char*)buf->iface.get_base(buf);
    w.buffer = x.buffer = y.buffer = buf;
    w.data = base + ow; x.data = base + ox; y.data = base + oy;
    buf->iface.clear(buf, 0);
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
    FILE* f = fopen(argv[8], "wb");
    CHECK(f && fwrite(out.data(), 1, out.size(), f) == out.size());
    fclose(f);

    // a graph with a node this backend cannot run is refused as a whole: the result buffer stays untouched
    bad.op = GGML_OP_ADD;
    bad.src[0] = &y;
    bad.src[1] = &y;
    bad.buffer = buf;
    bad.data = y.data;
    CHECK(!dev->iface.supports_op(dev, &bad));
    buf->iface.memset_tensor(buf, &y, 0xEE, 0, ggml_nbytes(&y));
    graph.n_nodes = 2;
    CHECK(backend->iface.graph_compute(backend, &graph) == GGML_STATUS_FAILED);
    std::vector<uint8_t> after(ggml_nbytes(&y));
    buf->iface.get_tensor(buf, &y, after.data(), 0, after.size());
    for (uint8_t v : after) CHECK(v == 0xEE);

    buf->iface.free_buffer(buf);
    delete buf;
    backend->iface.free(backend);
    printf("ok\n");
    return 0;
}
