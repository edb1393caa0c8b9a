// Host side of the C ABI: status reporting, the interval LUT, the bounded conversion
// cache with its workspaces, and the switched-linear dispatch
// (DynamicLinear._forward, kairos/dynamic_linear.py:131-172).
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

namespace kairos {

static thread_local std::string g_last_error;

int note_cuda_error(cudaError_t e) {
    g_last_error = std::string(cudaGetErrorName(e)) + ": " + cudaGetErrorString(e);
    cudaGetLastError();   // clear the sticky-free error state
    return KAIROS_ERR_CUDA;
}

static std::atomic<int>& arithmetic_word() {
    static std::atomic<int> rule([] {
        const char* v = std::getenv("KAIROS_ARITHMETIC");
        return (v && std::string(v) == "reference_cuda") ? (int)KAIROS_ARITH_REFERENCE_CUDA : (int)KAIROS_ARITH_TORCH;
    }());
    return rule;
}
int arithmetic_rule() { return arithmetic_word().load(std::memory_order_relaxed); }

bool chained_launch_enabled() {
    static const bool on = [] {
        const char* e = getenv("KAIROS_NO_PDL");
        return !(e && e[0] == '1');
    }();
    return on;
}

int launch_status() {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KAIROS_OK : note_cuda_error(e);
}

void set_last_error(const char* msg) { g_last_error = msg; }

static int fail(int code, const char* what) {
    g_last_error = what;
    return code;
}

// One host-mapped status word per device: kernels raise it when a bounded wait runs out;
// the host can read it without a copy.
int* device_status_word() {
    static int* words[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(mu);
    if (!words[dev]) {
        int* w = nullptr;
        if (cudaHostAlloc(reinterpret_cast<void**>(&w), sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) !=
            cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        *w = 0;
        words[dev] = w;
    }
    return words[dev];
}

size_t gemm_workspace_bytes(int M, int N, int K);   // gemm_sm100.cu
int noalloc_status(int clear);                       // gemm_sm100.cu: status word of kairos_w4a16_gemm_noalloc

struct Lut {
    std::vector<int> bounds;   // exclusive right ends of the intervals, ascending
    std::vector<int> ids;
    int memo_m = 0, memo_id = 0;
    bool memo_valid = false;
};

struct CacheEntry {
    const void* layer = nullptr;
    int bits = 0;               // 8 or 16
    int rule = 0;               // arithmetic rule the conversion ran under
    void* ptr = nullptr;
    size_t bytes = 0;
    uint64_t last_tick = 0;
    std::vector<cudaStream_t> users;   // every stream that was handed the pointer (its reads may still be queued)
    cudaEvent_t ready = nullptr;       // recorded after the conversion that filled the entry
    bool pinned = false;               // handed out while a stream was capturing: a graph holds the pointer
};

struct Ctx {
    size_t cache_limit = 0;
    size_t in_use = 0;
    uint64_t tick = 0, hits = 0, misses = 0, evictions = 0;
    std::vector<CacheEntry> entries;
    void* transient = nullptr;   // conversion target when the cache cannot hold the weight
    size_t transient_bytes = 0;
    std::vector<cudaStream_t> transient_users;   // streams whose queued work may still read `transient`
    void* act_ws = nullptr;      // Xq [M,K] int8 followed by sx [M] fp16
    size_t act_bytes = 0;
    void* gemm_ws = nullptr;     // split-K partial tiles
    size_t gemm_bytes = 0;
    // device staging for the host-buffer entry point: two input slots (the copy of call i+1 runs while call i
    // computes), one output buffer, copies on the context's own streams
    void* host_x[2] = {nullptr, nullptr};
    void* host_y = nullptr;
    size_t host_x_bytes[2] = {0, 0}, host_y_bytes = 0;
    cudaStream_t h2d = nullptr, d2h = nullptr;
    cudaEvent_t x_ready[2] = {nullptr, nullptr}, x_free[2] = {nullptr, nullptr}, y_ready = nullptr, y_done = nullptr;
    bool x_used[2] = {false, false};
    unsigned host_calls = 0;
    cudaEvent_t fence = nullptr;
    std::mutex mu;
};

struct Layer {
    Ctx* ctx;
    int N, K;
    const void *qweight, *scales, *scaled_zeros, *scales_to8, *scaled_zeros_to8, *scales_1, *bias;
};

static bool capturing(cudaStream_t st) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return cs != cudaStreamCaptureStatusNone;
}

// Grows a library-owned buffer.  Growth frees and allocates (an implicit device synchronisation), which a
// capturing stream must not see: inside a capture the buffers have to be large enough already
// (kairos_ctx_reserve, or an eager call of the same shape before the capture).
static int grow(void** ptr, size_t* have, size_t need, cudaStream_t st = nullptr, bool st_known = false) {
    if (*have >= need) return KAIROS_OK;
    if (st_known && capturing(st))
        return fail(KAIROS_ERR_WORKSPACE, "a library workspace would have to grow while the stream is capturing: call "
                                          "kairos_ctx_reserve (or run the same shape eagerly) before the capture");
    if (*ptr) KAIROS_CUDA_OK(cudaFree(*ptr));   // cudaFree waits for work that may still use the block
    *ptr = nullptr;
    *have = 0;
    size_t want = need + need / 4;
    want = (want + 255) & ~(size_t)255;
    KAIROS_CUDA_OK(cudaMalloc(ptr, want));
    *have = want;
    return KAIROS_OK;
}

static int ensure_gemm_ws(Ctx* c, int M, int N, int K, cudaStream_t st) {
    const size_t need = gemm_workspace_bytes(M, N, K);
    if (c->gemm_bytes >= need) return KAIROS_OK;
    return grow(&c->gemm_ws, &c->gemm_bytes, need, st, true);
}

static size_t act_ws_bytes(int M, int K) { return (((size_t)M * K + 255) & ~(size_t)255) + (size_t)M * 2 + 256; }

// Make `st` wait for everything the streams in `users` (other than `st`) have queued so far.  Calls on a
// context are serialised by its mutex, so whatever read the buffer has been enqueued by now.
static int order_after_users(Ctx* c, const std::vector<cudaStream_t>& users, cudaStream_t st) {
    for (cudaStream_t u : users) {
        if (u == st) continue;
        KAIROS_CUDA_OK(cudaEventRecord(c->fence, u));
        KAIROS_CUDA_OK(cudaStreamWaitEvent(st, c->fence, 0));
    }
    return KAIROS_OK;
}

static void note_user(std::vector<cudaStream_t>& users, cudaStream_t st) {
    if (std::find(users.begin(), users.end(), st) == users.end()) users.push_back(st);
}

// Returns the converted weight of `layer` in `bits` precision, converting on a miss.
// While `st` is capturing, nothing is evicted, freed or allocated: a miss fails with KAIROS_ERR_CACHE
// (convert eagerly first, e.g. kairos_layer_prefetch), and an entry handed to a capture is pinned --
// a graph may replay with its address -- until kairos_ctx_clear_cache.
static int converted_weight(Layer* L, int bits, cudaStream_t st, const void** out) {
    Ctx* c = L->ctx;
    const size_t bytes = (size_t)L->N * L->K * (bits == 8 ? 1 : 2);
    const bool cap = capturing(st);
    const int rule = arithmetic_rule();
    ++c->tick;
    for (auto& e : c->entries) {
        if (e.layer == L && e.bits == bits && e.rule == rule) {
            ++c->hits;
            e.last_tick = c->tick;
            if (std::find(e.users.begin(), e.users.end(), st) == e.users.end()) {
                // first use on this stream: order it after the conversion.  A capturing stream can neither wait
                // on an event recorded outside its capture nor let the host wait for it.
                if (cap)
                    return fail(KAIROS_ERR_CACHE, "the converted weight was produced on another stream and this stream is "
                                                  "capturing: run the layer once on this stream before the capture");
                KAIROS_CUDA_OK(cudaStreamWaitEvent(st, e.ready, 0));
                e.users.push_back(st);
            }
            if (cap) e.pinned = true;
            *out = e.ptr;
            return KAIROS_OK;
        }
    }
    // A weight the cache cannot hold at all is converted into the reusable slot on every call; that is a
    // plain kernel launch, so it may be captured -- provided the slot is already large enough.
    const bool uncacheable = bytes > c->cache_limit;
    if (cap && !(uncacheable && c->transient_bytes >= bytes))
        return fail(KAIROS_ERR_CACHE, "the converted weight is not in the cache and the stream is capturing: conversions "
                                      "allocate and evict, so run the layer (or kairos_layer_prefetch) eagerly before "
                                      "the capture, with a cache that holds every layer the graph uses");
    ++c->misses;
    void* dst = nullptr;
    CacheEntry* slot = nullptr;
    size_t evictable = 0;
    for (auto& e : c->entries)
        if (!e.pinned) evictable += e.bytes;
    if (bytes <= c->cache_limit && c->in_use - evictable + bytes <= c->cache_limit) {
        // evict least-recently-used entries until the new one fits; recycle an evicted block of the same size
        while (c->in_use + bytes > c->cache_limit) {
            size_t lru = c->entries.size();
            for (size_t i = 0; i < c->entries.size(); ++i)
                if (!c->entries[i].pinned && (lru == c->entries.size() || c->entries[i].last_tick < c->entries[lru].last_tick))
                    lru = i;
            if (lru == c->entries.size()) break;
            CacheEntry victim = c->entries[lru];
            c->entries.erase(c->entries.begin() + lru);
            c->in_use -= victim.bytes;
            ++c->evictions;
            if (!dst && victim.bytes == bytes) {
                const int rc = order_after_users(c, victim.users, st);
                if (rc != KAIROS_OK) return rc;
                dst = victim.ptr;
                cudaEventDestroy(victim.ready);
            } else {
                cudaEventDestroy(victim.ready);
                KAIROS_CUDA_OK(cudaFree(victim.ptr));   // waits for the work that may still read the block
            }
        }
        if (!dst) KAIROS_CUDA_OK(cudaMalloc(&dst, bytes));
        CacheEntry e;
        e.layer = L; e.bits = bits; e.rule = rule; e.ptr = dst; e.bytes = bytes; e.last_tick = c->tick;
        e.users.push_back(st);
        KAIROS_CUDA_OK(cudaEventCreateWithFlags(&e.ready, cudaEventDisableTiming));
        c->entries.push_back(e);
        c->in_use += bytes;
        slot = &c->entries.back();
    } else {
        // not cacheable: convert into the single reusable slot.  Its previous readers, on whatever stream,
        // were enqueued under the context's mutex before this call, so fencing those streams orders the reuse.
        int rc = order_after_users(c, c->transient_users, st);
        if (rc != KAIROS_OK) return rc;
        if ((rc = grow(&c->transient, &c->transient_bytes, bytes)) != KAIROS_OK) return rc;
        c->transient_users.clear();
        c->transient_users.push_back(st);
        dst = c->transient;
    }
    int rc;
    if (bits == 8)
        rc = kairos_w4_to_w8(L->qweight, L->scales_to8, L->scaled_zeros_to8, dst, L->N, L->K,
                             reinterpret_cast<kairos_stream_t>(st));
    else
        rc = kairos_w4_to_f16(L->qweight, L->scales, L->scaled_zeros, dst, L->N, L->K,
                              reinterpret_cast<kairos_stream_t>(st));
    if (rc != KAIROS_OK) return rc;
    if (slot) KAIROS_CUDA_OK(cudaEventRecord(slot->ready, st));
    *out = dst;
    return KAIROS_OK;
}

static int run_switched(Layer* L, const void* X, void* Y, int M, int comp, cudaStream_t st) {
    Ctx* c = L->ctx;
    kairos_stream_t ks = reinterpret_cast<kairos_stream_t>(st);
    if (M < 0) return KAIROS_ERR_SHAPE;
    if (M == 0) return KAIROS_OK;
    int rc;
    switch (comp) {
        case KAIROS_COMP_W4A16_GEMV:
            return kairos_w4a16_small_batch(X, L->qweight, L->scales, L->scaled_zeros, L->bias, Y, M, L->N, L->K, ks);
        case KAIROS_COMP_W4A16_GEMM:
            if ((rc = ensure_gemm_ws(c, M, L->N, L->K, st)) != KAIROS_OK) return rc;
            return kairos_w4a16_gemm(X, L->qweight, L->scales, L->scaled_zeros, L->bias, Y, M, L->N, L->K, c->gemm_ws,
                                     c->gemm_bytes, ks);
        case KAIROS_COMP_W8A8: {
            const void* w8 = nullptr;
            if ((rc = converted_weight(L, 8, st, &w8)) != KAIROS_OK) return rc;
            if ((rc = grow(&c->act_ws, &c->act_bytes, act_ws_bytes(M, L->K), st, true)) != KAIROS_OK) return rc;
            if ((rc = ensure_gemm_ws(c, M, L->N, L->K, st)) != KAIROS_OK) return rc;
            void* xq = c->act_ws;
            void* sx = static_cast<uint8_t*>(c->act_ws) + (((size_t)M * L->K + 255) & ~(size_t)255);
            if ((rc = kairos_act_quant_i8(X, xq, sx, M, L->K, ks)) != KAIROS_OK) return rc;
            return kairos_w8a8_gemm(xq, w8, L->scales_1, sx, L->bias, Y, nullptr, M, L->N, L->K, c->gemm_ws,
                                    c->gemm_bytes, ks);
        }
        case KAIROS_COMP_W8A16_GEMM: {
            const void* w8 = nullptr;
            if ((rc = converted_weight(L, 8, st, &w8)) != KAIROS_OK) return rc;
            if ((rc = ensure_gemm_ws(c, M, L->N, L->K, st)) != KAIROS_OK) return rc;
            return kairos_w8a16_gemm(X, w8, L->scales_1, L->bias, Y, M, L->N, L->K, c->gemm_ws, c->gemm_bytes, ks);
        }
        case KAIROS_COMP_FP16: {
            const void* w16 = nullptr;
            if ((rc = converted_weight(L, 16, st, &w16)) != KAIROS_OK) return rc;
            if ((rc = ensure_gemm_ws(c, M, L->N, L->K, st)) != KAIROS_OK) return rc;
            return kairos_f16_gemm(X, w16, L->bias, Y, M, L->N, L->K, c->gemm_ws, c->gemm_bytes, ks);
        }
        default:
            return fail(KAIROS_ERR_COMP, "kernel id is not one of 0 (w4a16_gemm), 1 (w4a16_gemv), 2 (w8a8), "
                                         "3 (w8a16_gemm), 5 (fp16)");
    }
}

}  // namespace kairos

using kairos::Ctx;
using kairos::Layer;
using kairos::Lut;

extern "C" {

int kairos_abi_version(void) { return 1; }

const char* kairos_status_str(int status) {
    switch (status) {
        case KAIROS_OK: return "ok";
        case KAIROS_ERR_SHAPE: return "shape rule violated (N % 4, K % 128, M range)";
        case KAIROS_ERR_ALIGN: return "null or misaligned pointer";
        case KAIROS_ERR_CUDA: return "CUDA call failed";
        case KAIROS_ERR_WORKSPACE: return "workspace missing or too small";
        case KAIROS_ERR_CACHE: return "conversion cache cannot hold the weight";
        case KAIROS_ERR_COMP: return "unknown kernel id";
        case KAIROS_ERR_DEVICE: return "a device-side wait ran out";
        case KAIROS_ERR_ARG: return "bad handle or argument";
        default: return "unknown status";
    }
}

const char* kairos_last_error(void) { return kairos::g_last_error.c_str(); }

int kairos_set_arithmetic(int rule) {
    if (rule != KAIROS_ARITH_TORCH && rule != KAIROS_ARITH_REFERENCE_CUDA) return KAIROS_ERR_ARG;
    return kairos::arithmetic_word().exchange(rule);
}
int kairos_get_arithmetic(void) { return kairos::arithmetic_rule(); }

/* Reads (and with clear != 0 resets) the status words of the current device: the host-mapped word the
 * kernels raise, and the word inside the library image that launches of kairos_w4a16_gemm_noalloc raise
 * (read with a plain copy, which synchronises the device).  Call after synchronising the stream(s) of
 * interest.  KAIROS_OK or KAIROS_ERR_DEVICE. */
int kairos_device_status(int clear) {
    int* w = kairos::device_status_word();
    if (!w) return KAIROS_ERR_CUDA;
    int v = *reinterpret_cast<volatile int*>(w);
    if (clear) *reinterpret_cast<volatile int*>(w) = 0;
    const int v2 = kairos::noalloc_status(clear);
    if (v == KAIROS_OK) v = v2;
    return v;
}

/* Kernel id 1 (w4a16_gemv) is served by two kernels: the warp-MMA decode kernel (N % 8 == 0), the
 * CUDA-core weight streamer otherwise (N % 8 == 4). */
int kairos_w4a16_small_batch(const void* X, const void* qweight, const void* scales, const void* scaled_zeros,
                             const void* bias, void* Y, int M, int N, int K, kairos_stream_t stream) {
    if (M <= 32 && (N % 8) == 0)
        return kairos_w4a16_decode(X, qweight, scales, scaled_zeros, bias, Y, M, N, K, stream);
    return kairos_w4a16_gemv(X, qweight, scales, scaled_zeros, bias, Y, M, N, K, stream);
}

// ------------------------------- LUT ---------------------------------------
kairos_lut* kairos_lut_create(void) { return reinterpret_cast<kairos_lut*>(new Lut()); }
void kairos_lut_destroy(kairos_lut* t) { delete reinterpret_cast<Lut*>(t); }

int kairos_lut_record(kairos_lut* t, int r, int comp_type) {
    if (!t) return KAIROS_ERR_ARG;
    Lut* l = reinterpret_cast<Lut*>(t);
    l->bounds.push_back(r + 1);   // interval (previous r, r] as a half-open [.., r+1)
    l->ids.push_back(comp_type);   // the memo is kept, as in lut.h: tables are filled before they are asked
    return KAIROS_OK;
}

int kairos_lut_get(kairos_lut* t, int m) {
    if (!t) return KAIROS_ERR_ARG;
    Lut* l = reinterpret_cast<Lut*>(t);
    if (l->ids.empty()) return KAIROS_ERR_ARG;
    if (l->memo_valid && m == l->memo_m) return l->memo_id;   // one-entry memo: a layer asks again only when M changed
    int id;
    if (m >= l->bounds.back()) {
        id = l->ids.back();                  // beyond the last profiled M: keep the last winner
    } else {
        const size_t i = std::upper_bound(l->bounds.begin(), l->bounds.end(), m) - l->bounds.begin();
        id = l->ids[i];
    }
    l->memo_m = m;
    l->memo_id = id;
    l->memo_valid = true;
    return id;
}

void kairos_lut_shrink_to_fit(kairos_lut* t) {
    if (!t) return;
    Lut* l = reinterpret_cast<Lut*>(t);
    l->bounds.shrink_to_fit();
    l->ids.shrink_to_fit();
}

int kairos_lut_size(const kairos_lut* t) { return t ? (int)reinterpret_cast<const Lut*>(t)->ids.size() : 0; }

// ------------------------------- context ------------------------------------
kairos_ctx* kairos_ctx_create(size_t cache_bytes) {
    Ctx* c = new Ctx();
    c->cache_limit = cache_bytes;
    if (cudaEventCreateWithFlags(&c->fence, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        delete c;
        return nullptr;
    }
    return reinterpret_cast<kairos_ctx*>(c);
}

void kairos_ctx_clear_cache(kairos_ctx* ctx) {
    if (!ctx) return;
    Ctx* c = reinterpret_cast<Ctx*>(ctx);
    std::lock_guard<std::mutex> lk(c->mu);
    for (auto& e : c->entries) {
        cudaFree(e.ptr);
        cudaEventDestroy(e.ready);
    }
    c->entries.clear();
    c->in_use = 0;
}

void kairos_ctx_destroy(kairos_ctx* ctx) {
    if (!ctx) return;
    kairos_ctx_clear_cache(ctx);
    Ctx* c = reinterpret_cast<Ctx*>(ctx);
    cudaFree(c->transient);
    cudaFree(c->act_ws);
    cudaFree(c->gemm_ws);
    cudaFree(c->host_x[0]);
    cudaFree(c->host_x[1]);
    cudaFree(c->host_y);
    if (c->h2d) cudaStreamDestroy(c->h2d);
    if (c->d2h) cudaStreamDestroy(c->d2h);
    for (int i = 0; i < 2; ++i) {
        if (c->x_ready[i]) cudaEventDestroy(c->x_ready[i]);
        if (c->x_free[i]) cudaEventDestroy(c->x_free[i]);
    }
    if (c->y_ready) cudaEventDestroy(c->y_ready);
    if (c->y_done) cudaEventDestroy(c->y_done);
    cudaEventDestroy(c->fence);
    cudaGetLastError();
    delete c;
}

int kairos_ctx_reserve(kairos_ctx* ctx, int max_M, int max_N, int max_K) {
    if (!ctx || max_M <= 0 || max_N <= 0 || max_K <= 0) return KAIROS_ERR_ARG;
    Ctx* c = reinterpret_cast<Ctx*>(ctx);
    std::lock_guard<std::mutex> lk(c->mu);
    int rc = kairos::grow(&c->act_ws, &c->act_bytes, kairos::act_ws_bytes(max_M, max_K));
    if (rc != KAIROS_OK) return rc;
    // the split-K scratch is largest for some M <= max_M; probe the token-tile boundaries
    size_t need = 0;
    const int probes[] = {16, 32, 64, 128, 256, 512, 1024, max_M};
    for (int m : probes)
        if (m <= max_M) need = std::max(need, kairos::gemm_workspace_bytes(m, max_N, max_K));
    return kairos::grow(&c->gemm_ws, &c->gemm_bytes, need);
}

int kairos_ctx_stats(const kairos_ctx* ctx, uint64_t* hits, uint64_t* misses, uint64_t* evictions,
                     uint64_t* bytes_in_use) {
    if (!ctx) return KAIROS_ERR_ARG;
    const Ctx* c = reinterpret_cast<const Ctx*>(ctx);
    if (hits) *hits = c->hits;
    if (misses) *misses = c->misses;
    if (evictions) *evictions = c->evictions;
    if (bytes_in_use) *bytes_in_use = c->in_use;
    return KAIROS_OK;
}

// ------------------------------- layer --------------------------------------
kairos_layer* kairos_layer_create(kairos_ctx* ctx, int N, int K, const void* qweight, const void* scales,
                                  const void* scaled_zeros, const void* scales_to8, const void* scaled_zeros_to8,
                                  const void* scales_1, const void* bias) {
    if (!ctx || N <= 0 || K <= 0 || (N % kairos::kInterleave) != 0 || (K % kairos::kGroup) != 0 || !qweight ||
        !scales || !scaled_zeros || !scales_to8 || !scaled_zeros_to8 || !scales_1) {
        kairos::fail(KAIROS_ERR_ARG, "kairos_layer_create: null tensor or N % 4 / K % 128 violated");
        return nullptr;
    }
    Layer* L = new Layer{reinterpret_cast<Ctx*>(ctx), N, K, qweight, scales, scaled_zeros, scales_to8,
                         scaled_zeros_to8, scales_1, bias};
    return reinterpret_cast<kairos_layer*>(L);
}

void kairos_layer_destroy(kairos_layer* layer) {
    if (!layer) return;
    Layer* L = reinterpret_cast<Layer*>(layer);
    Ctx* c = L->ctx;
    {
        std::lock_guard<std::mutex> lk(c->mu);
        for (size_t i = 0; i < c->entries.size();) {
            if (c->entries[i].layer == L) {
                cudaFree(c->entries[i].ptr);
                cudaEventDestroy(c->entries[i].ready);
                c->in_use -= c->entries[i].bytes;
                c->entries.erase(c->entries.begin() + i);
            } else {
                ++i;
            }
        }
    }
    delete L;
}

int kairos_switched_linear(kairos_layer* layer, const void* X, void* Y, int M, int comp_type,
                           kairos_stream_t stream) {
    if (!layer) return KAIROS_ERR_ARG;
    Layer* L = reinterpret_cast<Layer*>(layer);
    std::lock_guard<std::mutex> lk(L->ctx->mu);
    return kairos::run_switched(L, X, Y, M, comp_type, reinterpret_cast<cudaStream_t>(stream));
}

int kairos_switched_linear_q8(kairos_layer* layer, const void* Xq, const void* sx, void* Y, int M,
                              kairos_stream_t stream) {
    if (!layer) return KAIROS_ERR_ARG;
    if (M < 0) return KAIROS_ERR_SHAPE;
    if (M == 0) return KAIROS_OK;
    Layer* L = reinterpret_cast<Layer*>(layer);
    std::lock_guard<std::mutex> lk(L->ctx->mu);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const void* w8 = nullptr;
    int rc;
    if ((rc = kairos::converted_weight(L, 8, st, &w8)) != KAIROS_OK) return rc;
    if ((rc = kairos::ensure_gemm_ws(L->ctx, M, L->N, L->K, st)) != KAIROS_OK) return rc;
    return kairos_w8a8_gemm(Xq, w8, L->scales_1, sx, L->bias, Y, nullptr, M, L->N, L->K, L->ctx->gemm_ws,
                            L->ctx->gemm_bytes, stream);
}

int kairos_layer_prefetch(kairos_layer* layer, int comp_type, kairos_stream_t stream) {
    if (!layer) return KAIROS_ERR_ARG;
    Layer* L = reinterpret_cast<Layer*>(layer);
    std::lock_guard<std::mutex> lk(L->ctx->mu);
    const void* w = nullptr;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (comp_type == KAIROS_COMP_W8A8 || comp_type == KAIROS_COMP_W8A16_GEMM)
        return kairos::converted_weight(L, 8, st, &w);
    if (comp_type == KAIROS_COMP_FP16) return kairos::converted_weight(L, 16, st, &w);
    if (comp_type == KAIROS_COMP_W4A16_GEMM || comp_type == KAIROS_COMP_W4A16_GEMV) return KAIROS_OK;
    return KAIROS_ERR_COMP;
}

int kairos_switched_linear_host(kairos_layer* layer, const void* X_host, void* Y_host, int M, int comp_type,
                                kairos_stream_t stream) {
    if (!layer || !X_host || !Y_host) return KAIROS_ERR_ARG;
    if (M < 0) return KAIROS_ERR_SHAPE;
    if (M == 0) return KAIROS_OK;
    Layer* L = reinterpret_cast<Layer*>(layer);
    Ctx* c = L->ctx;
    std::lock_guard<std::mutex> lk(c->mu);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const size_t xb = (size_t)M * L->K * 2, yb = (size_t)M * L->N * 2;
    int rc;
    if (!c->h2d) {
        KAIROS_CUDA_OK(cudaStreamCreateWithFlags(&c->h2d, cudaStreamNonBlocking));
        KAIROS_CUDA_OK(cudaStreamCreateWithFlags(&c->d2h, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            KAIROS_CUDA_OK(cudaEventCreateWithFlags(&c->x_ready[i], cudaEventDisableTiming));
            KAIROS_CUDA_OK(cudaEventCreateWithFlags(&c->x_free[i], cudaEventDisableTiming));
        }
        KAIROS_CUDA_OK(cudaEventCreateWithFlags(&c->y_ready, cudaEventDisableTiming));
        KAIROS_CUDA_OK(cudaEventCreateWithFlags(&c->y_done, cudaEventDisableTiming));
    }
    const int slot = (int)(c->host_calls++ & 1u);
    if ((rc = kairos::grow(&c->host_x[slot], &c->host_x_bytes[slot], xb)) != KAIROS_OK) return rc;
    if ((rc = kairos::grow(&c->host_y, &c->host_y_bytes, yb)) != KAIROS_OK) return rc;
    // input copy on its own stream: it may run while the previous call still computes or copies out
    if (c->x_used[slot]) KAIROS_CUDA_OK(cudaStreamWaitEvent(c->h2d, c->x_free[slot], 0));   // the call two back has read the slot
    KAIROS_CUDA_OK(cudaMemcpyAsync(c->host_x[slot], X_host, xb, cudaMemcpyHostToDevice, c->h2d));
    KAIROS_CUDA_OK(cudaEventRecord(c->x_ready[slot], c->h2d));
    KAIROS_CUDA_OK(cudaStreamWaitEvent(st, c->x_ready[slot], 0));
    if ((rc = kairos::run_switched(L, c->host_x[slot], c->host_y, M, comp_type, st)) != KAIROS_OK) return rc;
    KAIROS_CUDA_OK(cudaEventRecord(c->x_free[slot], st));
    c->x_used[slot] = true;
    KAIROS_CUDA_OK(cudaEventRecord(c->y_ready, st));
    // output copy on its own stream; `stream` waits for it, so the result is there once `stream` is synchronized
    KAIROS_CUDA_OK(cudaStreamWaitEvent(c->d2h, c->y_ready, 0));
    KAIROS_CUDA_OK(cudaMemcpyAsync(Y_host, c->host_y, yb, cudaMemcpyDeviceToHost, c->d2h));
    KAIROS_CUDA_OK(cudaEventRecord(c->y_done, c->d2h));
    KAIROS_CUDA_OK(cudaStreamWaitEvent(st, c->y_done, 0));
    return KAIROS_OK;
}

}  // extern "C"
