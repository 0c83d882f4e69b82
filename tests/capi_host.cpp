// A host program without a line of Python: loads the C handle API, builds an engine with random weights from a preset,
// generates greedily and prints the ids; then runs two steps by hand and prints the argmax of each row of logits.
// Built and run by tests/test_capi_gpu.py (g++ capi_host.cpp -Wl,--no-as-needed -lpython3.12 -ldl).
#include <dlfcn.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

struct ib_engine;
using create_t = ib_engine* (*)(const char*, const char*, uint64_t, const char*, int, int, int, int);
using destroy_t = void (*)(ib_engine*);
using vocab_t = int64_t (*)(ib_engine*);
using req_t = int (*)(ib_engine*, int64_t);
using step_t = int64_t (*)(ib_engine*, int, const int64_t*, const int32_t*, const int32_t*, const int32_t*, const int32_t*, int32_t*);
using logits_t = int64_t (*)(ib_engine*, float*, int64_t);
using gen_t = int (*)(ib_engine*, int, const int32_t*, const int32_t*, int, float, uint64_t, int64_t, int32_t*, int32_t*);
using err_t = const char* (*)(void);

int main(int argc, char** argv) {
    if (argc < 3) { std::fprintf(stderr, "usage: capi_host <library> <preset>\n"); return 2; }
    void* lib = dlopen(argv[1], RTLD_NOW | RTLD_GLOBAL);
    if (!lib) { std::fprintf(stderr, "dlopen: %s\n", dlerror()); return 1; }
    auto create = (create_t)dlsym(lib, "ib_engine_create");
    auto destroy = (destroy_t)dlsym(lib, "ib_engine_destroy");
    auto vocab = (vocab_t)dlsym(lib, "ib_engine_vocab_size");
    auto add = (req_t)dlsym(lib, "ib_engine_add_request");
    auto end = (req_t)dlsym(lib, "ib_engine_end_request");
    auto step = (step_t)dlsym(lib, "ib_engine_step");
    auto logits = (logits_t)dlsym(lib, "ib_engine_get_logits");
    auto gen = (gen_t)dlsym(lib, "ib_engine_generate");
    auto err = (err_t)dlsym(lib, "ib_api_last_error");
    if (!create || !destroy || !vocab || !add || !end || !step || !logits || !gen || !err) { std::fprintf(stderr, "missing symbol\n"); return 1; }
    ib_engine* e = create(nullptr, argv[2], 4, "float32", 2, 64, 0, 16);
    if (!e) { std::fprintf(stderr, "create: %s\n", err()); return 1; }
    const int32_t prompt[] = {3, 200, 17, 42, 9, 9, 101};
    const int32_t lens[] = {7};
    int32_t out[8], got[1];
    if (gen(e, 1, lens, prompt, 8, 0.0f, 0, -1, out, got)) { std::fprintf(stderr, "generate: %s\n", err()); return 1; }
    std::printf("generated");
    for (int i = 0; i < got[0]; i++) std::printf(" %d", out[i]);
    std::printf("\n");
    // the same by hand: the prompt as one step, then one token
    const int64_t V = vocab(e);
    const int64_t ids[] = {5};
    const int32_t n_tokens[] = {7}, n_want[] = {2}, want[] = {0, 6};
    if (add(e, 5)) { std::fprintf(stderr, "add: %s\n", err()); return 1; }
    int64_t rows = step(e, 1, ids, n_tokens, prompt, n_want, want, nullptr);
    if (rows != 2) { std::fprintf(stderr, "step: %lld %s\n", (long long)rows, err()); return 1; }
    std::vector<float> buf(size_t(rows * V));
    if (logits(e, buf.data(), int64_t(buf.size())) != rows) { std::fprintf(stderr, "logits: %s\n", err()); return 1; }
    std::printf("argmax");
    for (int64_t r = 0; r < rows; r++) {
        int64_t best = 0;
        for (int64_t v = 1; v < V; v++) if (buf[size_t(r * V + v)] > buf[size_t(r * V + best)]) best = v;
        std::printf(" %lld", (long long)best);
    }
    std::printf("\n");
    // an unknown request is an error with a message, not a crash
    const int64_t bad[] = {99};
    const int32_t one[] = {1}, zero[] = {0}, tok[] = {1};
    if (step(e, 1, bad, one, tok, zero, nullptr, nullptr) >= 0) { std::fprintf(stderr, "a step for an unknown request succeeded\n"); return 1; }
    std::printf("error %s\n", err());
    end(e, 5);
    destroy(e);
    return 0;
}
