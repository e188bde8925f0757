// Library-wide state: last-error text, per-thread stream, per-device scratch,
// the math-mode switch and the launch counter.
#include "common.cuh"
#include <atomic>
#include <mutex>
#include <cstring>
#include <cstdlib>

namespace bmb {

static thread_local char g_err[512] = "";
static thread_local cudaStream_t g_stream = 0;
static std::atomic<long long> g_launches{0};
static std::atomic<int> g_math{-1};

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    if (getenv("BMB_VERBOSE")) fprintf(stderr, "bmb: error %d: %s\n", code, g_err);
    return code;
}

cudaStream_t cur_stream() { return g_stream; }

static thread_local bool g_emit_rounded = false;
bool emit_rounded() { return g_emit_rounded; }
void set_emit_rounded(bool on) { g_emit_rounded = on; }

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launches_total() { return g_launches.load(std::memory_order_relaxed); }

int current_device() {
    int d = 0;
    cudaGetDevice(&d);
    return d;
}

int sm_count() {
    static int cache[64];
    static std::once_flag once;
    std::call_once(once, [] { for (int &c : cache) c = 0; });
    const int d = current_device();
    if (d < 0 || d >= 64) return 148;
    if (cache[d] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0) n = 148;
        cache[d] = n;
    }
    return cache[d];
}

struct Scratch { void *p = nullptr; size_t cap = 0; };
static Scratch g_scratch[64][SCR_SLOTS];
static std::mutex g_scratch_mu;
static std::atomic<unsigned long long> g_scratch_gen[64];

unsigned long long scratch_generation() {
    const int d = current_device();
    return (d < 0 || d >= 64) ? 0ULL : g_scratch_gen[d].load(std::memory_order_relaxed);
}

void *device_scratch(ScratchSlot slot, size_t bytes) {
    const int d = current_device();
    if (d < 0 || d >= 64) { fail(BMB_E_ARG, "device index %d out of range", d); return nullptr; }
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    Scratch &s = g_scratch[d][slot];
    if (s.cap >= bytes && s.p) return s.p;
    // Growing: earlier work on this device may still read the old block.  Anything that has
    // remembered the old address (a captured CUDA graph) learns of the move from the generation count.
    if (s.p) { cudaDeviceSynchronize(); cudaFree(s.p); s.p = nullptr; s.cap = 0; }
    g_scratch_gen[d].fetch_add(1, std::memory_order_relaxed);
    size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) { fail(BMB_E_CUDA, "scratch cudaMalloc(%zu) -> %s", want, cudaGetErrorString(e)); return nullptr; }
    s.p = p; s.cap = want;
    return p;
}

// Who used a scratch slot last.  A caller about to overwrite a slot from another stream than its last user first
// makes its stream wait for that user's last kernel, so that two streams of one device take turns instead of racing.
// (Not while a stream is being captured: the captured launches carry their own order, and an event recorded inside a
// capture cannot be waited for outside it.)
struct SlotUse { cudaStream_t stream = nullptr; cudaEvent_t done = nullptr; bool valid = false; };
static SlotUse g_slot_use[64][SCR_SLOTS];

static bool capturing(cudaStream_t st) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) { cudaGetLastError(); return false; }
    return cs != cudaStreamCaptureStatusNone;
}

int scratch_acquire(ScratchSlot slot, cudaStream_t st) {
    const int d = current_device();
    if (d < 0 || d >= 64 || capturing(st)) return BMB_OK;
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    SlotUse &u = g_slot_use[d][slot];
    if (u.valid && u.stream != st) BMB_CUDA(cudaStreamWaitEvent(st, u.done, 0));
    return BMB_OK;
}

int scratch_release(ScratchSlot slot, cudaStream_t st) {
    const int d = current_device();
    if (d < 0 || d >= 64 || capturing(st)) return BMB_OK;
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    SlotUse &u = g_slot_use[d][slot];
    if (!u.done) BMB_CUDA(cudaEventCreateWithFlags(&u.done, cudaEventDisableTiming));
    BMB_CUDA(cudaEventRecord(u.done, st));
    u.stream = st;
    u.valid = true;
    return BMB_OK;
}

}  // namespace bmb

extern "C" {

const char *bmb_last_error(void) { return bmb::g_err; }
long long bmb_launch_count(void) { return bmb::launches_total(); }
const char *bmb_version(void) { return "bmb-b200 0.1 (sm_100a)"; }

int bmb_set_stream(void *s) { bmb::g_stream = (cudaStream_t)s; return BMB_OK; }
void *bmb_get_stream(void) { return (void *)bmb::g_stream; }

int bmb_set_math_mode(int mode) {
    if (mode < BMB_MATH_FP32 || mode > BMB_MATH_BF16)
        return bmb::fail(BMB_E_ARG, "math mode %d unknown", mode);
    bmb::g_math.store(mode);
    return BMB_OK;
}

int bmb_get_math_mode(void) {
    int m = bmb::g_math.load();
    if (m < 0) {
        // Default: fp32, the reference's arithmetic; BMB_MATH=tf32|bf16 opts in.
        m = BMB_MATH_FP32;
        const char *e = getenv("BMB_MATH");
        if (e && !strcmp(e, "tf32")) m = BMB_MATH_TF32;
        if (e && !strcmp(e, "bf16")) m = BMB_MATH_BF16;
        bmb::g_math.store(m);
    }
    return m;
}

}  // extern "C"
