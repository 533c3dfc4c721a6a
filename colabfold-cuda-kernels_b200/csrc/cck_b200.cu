// libcolabfold_cuda_kernels.so for B200: the diffusion sampler's C entry points.
//   cck_mk_sample        the operator core: what the XLA FFI handler MkSample wraps
//   mk_workspace_bytes   workspace size for a shape bucket
//   mk_*                 the stand-alone debug API (ctypes), same signatures as the reference's
// Declarations with the reference interfaces they replace: include/cck_b200.h.
#include "host.cuh"

using namespace cck;

namespace {

struct State {
    bool ready = false;
    Template t{};
    std::vector<void*> in;
    char* ws = nullptr;
    int* ext = nullptr;
    unsigned long long* timing = nullptr;
    Device dev;
    Control last{};
    int real_n = 0, real_ns = 0; // mk_set_extent: the real extents inside the bucket, 0 = the bucket's
};
State g_state;

__global__ void __launch_bounds__(kThreads, 1) gemm_test_kernel(const __grid_constant__ Launch L, const GemmDesc g) {
    for (int i = threadIdx.x; i < int(sizeof(KP) / 4); i += kThreads) { // the CTA's copy of the parameter block (wait limit, control words)
        reinterpret_cast<uint32_t*>(smem_base() + kKpOff)[i] = reinterpret_cast<const uint32_t*>(&L.kp)[i];
    }
    __syncthreads();
    gemm_init();
    if (threadIdx.x == 0) {
        GemmDesc t = g;
        gd_finish(t);
        gd_table()[0] = t;
    }
    __syncthreads();
    Run& r = *new (smem_base() + kRunOff + threadIdx.x * kRunSlot) Run();
    run_gemm(L, r, r.d, 0, 0, 0);
    __syncthreads();
    if (threadIdx.x == 0 && smem_ctl()->abort) {
        fail_launch(ST_PIPE_TIMEOUT, 0);
    }
    gemm_fini();
}

// One CTA, one thread waiting on an mbarrier that nothing arrives at, with the launch's (shortened)
// limit: the wait must give up, record the failure and let the kernel end normally.
__global__ void wait_test_kernel(Control* ctl, long long limit) {
    KP* p = reinterpret_cast<KP*>(smem_base() + kKpOff);
    SmemCtl* sc = smem_ctl();
    if (threadIdx.x == 0) {
        p->ctl = ctl, p->wait_cycles = limit;
        sc->abort = 0;
        mbar_init(&sc->full[0], 1);
        fence_mbar_init();
        const bool done = mbar_wait(&sc->full[0], 0, &sc->abort);
        if (!done && sc->abort) {
            fail_launch(ST_PIPE_TIMEOUT, 0);
        }
    }
}
// the sampler's Philox words and normals for one counter
__global__ void philox_test_kernel(uint32_t idx, uint32_t step, uint32_t sample, uint32_t stream, uint32_t k0, uint32_t k1,
                                   uint32_t* words, float* z) {
    const PhiloxWords c = philox(idx, step, sample, stream, k0, k1);
    const Normals4 n = philox_normals(idx, step, sample, stream, k0, k1);
    for (int i = 0; i < 4; i++) {
        words[i] = c.w[i], z[i] = n.z[i];
    }
}

} // namespace

extern "C" {

const char* cck_last_error() {
    return g_error.c_str();
}

// The operator: enqueue one whole sampling run on `stream`. All pointers are device pointers owned
// by the caller; nothing is allocated, freed or synchronised here.
int cck_mk_sample(void* stream, const int* ext, const void* const* in, const size_t* bytes, int num_inputs, float* out,
                  int out_tokens, void* ws, size_t ws_bytes, int samples, int nsteps, int flags) {
    if (num_inputs != kNumInputs) {
        return fail(E_ARITY, "MkSample: wrong number of inputs");
    }
    const int nsb = int(bytes[IN_QMASK] / sizeof(float) / kSubset);
    Template t;
    if (int e = make_template(t, samples, out_tokens, nsb, nsteps, uint32_t(flags), bytes)) {
        return e;
    }
    if (ws_bytes < t.total) {
        return fail(E_WORKSPACE, "MkSample: workspace too small");
    }
    Device dev;
    if (int e = device_state(dev)) {
        return e;
    }
    Launch L;
    if (int e = make_launch(L, t, dev, in, static_cast<char*>(ws), out, ext)) {
        return e;
    }
    L.kp.mode = 0;
    return enqueue(L, dev, static_cast<cudaStream_t>(stream));
}

// ---- the operator without a caller-supplied workspace
//
// XLA calls the operator on its own stream, often while it records a command buffer (a CUDA
// graph), and a C caller may sit inside a capture of its own. Neither can call cudaMalloc there:
// allocation is not a stream operation and is refused during capture, and XLA expects a handler
// to touch only the buffers it was handed. A caller that binds the operator without the workspace
// result therefore has no scratch to give. For such callers the library carries a fixed scratch
// array in device memory, reserved on every GPU that loads the library until the process exits.
constexpr size_t kStaticWsBytes = size_t(32) << 20; // 32 MiB: small folds only (e.g. 32 tokens, 1 sample)
static __device__ __align__(256) unsigned char g_static_ws[kStaticWsBytes];
static void* g_static_ws_ptr[kMaxDevices]; // the array's device address, per device ordinal
static std::mutex g_static_ws_mutex;

// Same arguments and result as cck_mk_sample, minus the workspace: the scratch is the library's
// built-in array. Calls no cudaMalloc, cudaFree or any allocating routine.
//  - Sizes: a fold that needs more than cck_static_workspace_bytes() of scratch is refused with
//    CCK_E_WORKSPACE and a message naming both sizes; use cck_mk_sample with your own workspace then.
//  - First call on a device: looks up the array's device address (once per device, with that
//    device current). Make this first call outside any stream capture.
//  - Every call on a device shares the one array, which keeps the previous call's contents. The
//    control words are cleared on the stream at the start of each call and every other buffer is
//    written before it is read, so calls one after another on a stream are independent. Two calls
//    that overlap on the GPU (different streams, no ordering between them) race on the array and
//    give wrong results: order them.
int cck_mk_sample_static(void* stream, const int* ext, const void* const* in, const size_t* bytes, int num_inputs,
                         float* out, int out_tokens, int samples, int nsteps, int flags) {
    if (num_inputs != kNumInputs) {
        return fail(E_ARITY, "MkSample: wrong number of inputs");
    }
    const int nsb = int(bytes[IN_QMASK] / sizeof(float) / kSubset);
    Template t;
    if (int e = make_template(t, samples, out_tokens, nsb, nsteps, uint32_t(flags), bytes)) {
        return e;
    }
    if (t.total > kStaticWsBytes) {
        return fail(E_WORKSPACE, "MkSample: this fold needs " + std::to_string(t.total) +
                                     " bytes of scratch, the built-in scratch holds " + std::to_string(kStaticWsBytes) +
                                     "; call cck_mk_sample with a workspace instead");
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        return fail(E_DEVICE, "MkSample: no CUDA device");
    }
    void* ws = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_ws_mutex);
        if (!g_static_ws_ptr[dev]) {
            // in host code the array's name is only a handle: the device address comes from the runtime
            void* ptr = nullptr;
            const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_ws);
            if (err != cudaSuccess || !ptr) {
                return fail(E_DEVICE, std::string("MkSample: built-in scratch: ") + cudaGetErrorString(err));
            }
            g_static_ws_ptr[dev] = ptr;
        }
        ws = g_static_ws_ptr[dev];
    }
    return cck_mk_sample(stream, ext, in, bytes, num_inputs, out, out_tokens, ws, kStaticWsBytes, samples, nsteps, flags);
}

size_t cck_static_workspace_bytes() {
    return kStaticWsBytes;
}

size_t mk_workspace_bytes(int S, int Nb, int NSb, int nsteps, int flags, const size_t* bytes) {
    Template t;
    if (make_template(t, S, Nb, NSb, nsteps, uint32_t(flags), bytes)) {
        return 0;
    }
    return t.total;
}

void mk_teardown() {
    for (void* p : g_state.in) {
        cudaFree(p);
    }
    cudaFree(g_state.ws), cudaFree(g_state.ext), cudaFree(g_state.timing);
    g_state = State{};
}

int mk_setup(int S, int N, int A, int NS, int steps, const void** host, const size_t* bytes) {
    mk_teardown();
    (void)A;
    const uint32_t flags = uint32_t(static_cast<const float*>(host[IN_MISC])[M_FLAGS]);
    if (make_template(g_state.t, S, N, NS, steps, flags, bytes)) {
        fprintf(stderr, "mk_setup: %s\n", g_error.c_str());
        return 1;
    }
    if (device_state(g_state.dev)) {
        fprintf(stderr, "mk_setup: %s\n", g_error.c_str());
        return 1;
    }
    g_state.in.assign(kNumInputs, nullptr);
    for (int i = 0; i < kNumInputs; i++) {
        if (cudaMalloc(&g_state.in[i], bytes[i] ? bytes[i] : 16) != cudaSuccess ||
            cudaMemcpy(g_state.in[i], host[i], bytes[i], cudaMemcpyHostToDevice) != cudaSuccess) {
            fprintf(stderr, "mk_setup: input %d: %s\n", i, cudaGetErrorString(cudaGetLastError()));
            return 1;
        }
    }
    if (cudaMalloc(&g_state.ws, g_state.t.total) != cudaSuccess || cudaMalloc(&g_state.ext, 5 * sizeof(int)) != cudaSuccess ||
        cudaMalloc(&g_state.timing, 2 * kKinds * sizeof(unsigned long long)) != cudaSuccess) {
        fprintf(stderr, "mk_setup: workspace of %zu bytes: %s\n", g_state.t.total, cudaGetErrorString(cudaGetLastError()));
        return 1;
    }
    cudaMemset(g_state.ws, 0, g_state.t.total);
    if (getenv("MK_VERBOSE")) {
        printf("mk: %d CTAs of %d threads, %d B shared memory per CTA; workspace %zu MB\n", g_state.dev.sms, kThreads,
               kSmemAlloc, g_state.t.total >> 20);
    }
    g_state.ready = true;
    return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// The real extents of the next runs inside the bucket given to mk_setup (tokens, 32-atom subsets);
// 0, 0 restores the bucket's. The reference's debug API always runs the bucket's extents; its
// operator takes the real ones from ext, which is what this setter feeds.
int mk_set_extent(int N, int NS) {
    if (!g_state.ready || N < 0 || NS < 0 || N > g_state.t.Nb || NS > g_state.t.NSb) {
        return 1;
    }
    g_state.real_n = N, g_state.real_ns = NS;
    return 0;
}

// 1 (default): the chains QKVG -> attention -> WO and W1 -> W2 of a token block run on completion
// counters; 0: on grid barriers, phase by phase as the reference's schedule (the per-kind timing
// record then splits them). Returns the previous setting.
int mk_set_flow(int on) {
    const int was = g_flow;
    g_flow = on != 0;
    return was;
}

// Test hook: the token attention's second pipeline starts `cycles` SM cycles (plus a few per CTA)
// after the first in every attention phase of the following runs; 0 (the default) switches it off.
// Results must not depend on it. Returns the previous setting.
int mk_set_attn_skew(int cycles) {
    const int was = g_attn_skew;
    g_attn_skew = cycles > 0 ? cycles : 0;
    return was;
}

// Test hook for the waits that give up: the following runs use `cycles` SM cycles as the limit of
// every wait (0: the default of about a second), and their grid barriers expect `extra` arrivals that
// no CTA makes, so that with extra > 0 the first barrier runs out. Such a run ends normally with
// status 1 (mk_run returns 1, cck_last_status tells). mk_set_wait_test(0, 0) restores production.
int mk_set_wait_test(long long cycles, int extra) {
    g_wait_cycles = cycles > 0 ? cycles : 0, g_barrier_extra = extra > 0 ? extra : 0;
    return 0;
}
// One thread waits `cycles` SM cycles on an mbarrier that nothing arrives at. Returns the status word
// the kernel left (2 = the wait gave up, as it must), or -1 on a CUDA error; *ms gets the launch time.
int mk_wait_test(long long cycles, float* ms) {
    Device dev;
    Control* ctl = nullptr;
    if (device_state(dev) || cudaMalloc(&ctl, sizeof(Control)) != cudaSuccess || cudaMemset(ctl, 0, sizeof(Control)) != cudaSuccess) {
        cudaFree(ctl);
        return -1;
    }
    cudaFuncSetAttribute(reinterpret_cast<const void*>(wait_test_kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAlloc);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0), cudaEventCreate(&e1);
    cudaEventRecord(e0);
    wait_test_kernel<<<1, 32, kSmemAlloc>>>(ctl, cycles);
    cudaEventRecord(e1);
    const cudaError_t err = cudaDeviceSynchronize();
    float el = 0.f;
    cudaEventElapsedTime(&el, e0, e1);
    if (ms) {
        *ms = el;
    }
    Control c{};
    cudaMemcpy(&c, ctl, sizeof c, cudaMemcpyDeviceToHost);
    cudaEventDestroy(e0), cudaEventDestroy(e1);
    cudaFree(ctl);
    return err == cudaSuccess ? int(c.status) : -1;
}
// The sampler's Philox4x32-10 words and Box-Muller normals for counter (idx, step, sample, stream) and
// key = seed, computed on the device (reference: src/diffusion/rng.cuh:14-46). 0 on success.
int mk_philox_test(uint32_t idx, uint32_t step, uint32_t sample, uint32_t stream, uint64_t seed, uint32_t* words, float* z) {
    uint32_t* dw = nullptr;
    float* dz = nullptr;
    if (cudaMalloc(&dw, 16) != cudaSuccess || cudaMalloc(&dz, 16) != cudaSuccess) {
        cudaFree(dw), cudaFree(dz);
        return 1;
    }
    philox_test_kernel<<<1, 1>>>(idx, step, sample, stream, uint32_t(seed), uint32_t(seed >> 32), dw, dz);
    const bool ok = cudaDeviceSynchronize() == cudaSuccess && cudaMemcpy(words, dw, 16, cudaMemcpyDeviceToHost) == cudaSuccess &&
                    cudaMemcpy(z, dz, 16, cudaMemcpyDeviceToHost) == cudaSuccess;
    cudaFree(dw), cudaFree(dz);
    return ok ? 0 : 1;
}

int mk_set_grid(int) {
    return g_state.dev.sms; // one CTA per SM, always
}

int mk_run(int mode, int nsteps, int dbg_stop, uint64_t seed, const float* xn, float t, float* ms,
           unsigned long long* timing) {
    State& s = g_state;
    if (!s.ready) {
        fprintf(stderr, "mk_run: mk_setup has not run\n");
        return 1;
    }
    const int ext[5] = {s.real_n ? s.real_n : s.t.Nb, s.real_ns ? s.real_ns : s.t.NSb, 1, int(uint32_t(seed)),
                        int(uint32_t(seed >> 32))};
    cudaMemcpy(s.ext, ext, sizeof ext, cudaMemcpyHostToDevice);
    Launch L;
    if (make_launch(L, s.t, s.dev, s.in.data(), s.ws, nullptr, s.ext)) {
        fprintf(stderr, "mk_run: %s\n", g_error.c_str());
        return 1;
    }
    L.kp.mode = mode, L.kp.nsteps = mode == 0 ? nsteps : 0, L.kp.t = t, L.kp.dbg_stop = dbg_stop;
    if (dbg_stop > 0) {
        L.kp.flow = 0; // a stop counts the barriers of the reference's schedule
    }
    make_program(L.prog, mode, L.kp.nsteps, s.t.flags | (L.kp.flow ? kProgFlow : 0));
    if (mode == 0 && nsteps > s.t.steps) {
        fprintf(stderr, "mk_run: %d steps, but SIGMA holds %d\n", nsteps, s.t.steps);
        return 1;
    }
    if (mode == 1) {
        cudaMemcpy(s.ws + s.t.off[B_XN], xn, s.t.bytes[B_XN], cudaMemcpyHostToDevice);
    }
    if (timing) {
        cudaMemset(s.timing, 0, 2 * kKinds * sizeof(unsigned long long));
        L.kp.timing = s.timing;
    }
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0), cudaEventCreate(&e1);
    cudaEventRecord(e0);
    const int rc = enqueue(L, s.dev, 0);
    cudaEventRecord(e1);
    cudaEventSynchronize(e1);
    float el = 0.f;
    cudaEventElapsedTime(&el, e0, e1);
    if (ms) {
        *ms = el;
    }
    cudaEventDestroy(e0), cudaEventDestroy(e1);
    const cudaError_t err = cudaDeviceSynchronize();
    if (rc || err != cudaSuccess) {
        fprintf(stderr, "mk_run: %s\n", rc ? g_error.c_str() : cudaGetErrorString(err));
        return 1;
    }
    if (timing) {
        cudaMemcpy(timing, s.timing, 2 * kKinds * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
    }
    cudaMemcpy(&s.last, s.ws, sizeof(Control), cudaMemcpyDeviceToHost);
    if (s.last.status != ST_OK) {
        fprintf(stderr, "mk_run: the kernel gave up (status %u at barrier %u)\n", s.last.status, s.last.where);
        return 1;
    }
    return 0;
}

// status word and barrier count of the last mk_run
void cck_last_status(unsigned int* status, unsigned int* where, unsigned int* barriers) {
    *status = g_state.last.status, *where = g_state.last.where;
    *barriers = g_state.dev.sms ? g_state.last.barrier / g_state.dev.sms : 0;
}

#if CCK_STAGE_REC
// diagnostics build only: per phase kind, the sums over CTAs and phases of the seven stamps (ns after
// the phase began) and the number of (CTA, phase) samples; reading clears the record
void mk_stage_rec(unsigned long long* out) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, g_stage_rec, sizeof(unsigned long long) * 32 * 16);
    static unsigned long long zero[32 * 16];
    cudaMemcpyToSymbol(g_stage_rec, zero, sizeof(zero));
}
#endif
#if CCK_TRACE
// diagnostics build only: the traced CTA's event records, [7 roles][2048] words of cycle << 16 | event << 8
// | value, and how many each role wrote; reading clears the counts
void mk_trace(unsigned long long* out, unsigned int* n) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, g_trace, sizeof(unsigned long long) * kTraceRoles * kTraceSlots);
    cudaMemcpyFromSymbol(n, g_trace_n, sizeof(unsigned int) * kTraceRoles);
    const unsigned int zero[kTraceRoles] = {};
    cudaMemcpyToSymbol(g_trace_n, zero, sizeof(zero));
}
// every CTA's wait at the first 1024 grid barriers of the last launch: [barrier][160] words of cycles | kind << 24
void mk_barrier_waits(unsigned int* out) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, g_barwait, sizeof(unsigned int) * kBarWaitSlots * 160);
}
#endif
// The phase program the host would hand to the kernel for (mode, nsteps, flags): up to max_ops
// operations as bytes {function, argument, block, end | kind << 2}. Returns the number of operations
// of the program, or -1. Needs no device.
int mk_program(int mode, int nsteps, int flags, unsigned char* ops, int max_ops) {
    static Program pr;
    if (make_program(pr, mode, nsteps, uint32_t(flags))) {
        return -1;
    }
    int n = 0;
    while (n < kMaxOps && pr.ops[n].fn != FN_END) {
        n++;
    }
    // the denoiser subroutine follows the main program's end
    int total = n + 1;
    while (total < kMaxOps && pr.ops[total - 1].fn != FN_RET) {
        total++;
    }
    for (int i = 0; i < total && i < max_ops; i++) {
        memcpy(ops + 4 * i, &pr.ops[i], 4);
    }
    return total;
}

// the phase kinds of mk_run's timing record, comma-separated: per kind [wall ns, phases]
const char* mk_timing_names() {
#define CCK_NAME(name) #name ","
    static const char names[] = CCK_KINDS(CCK_NAME);
#undef CCK_NAME
    return names;
}

// 2: atom adaLN modulations and atom pair logits arrive as f32
int mk_version() {
    return 2;
}

int mk_buf_id(const char* name) {
    for (int b = 0; b < kNumBufs; b++) {
        if (!strcmp(name, kBufNames[b])) {
            return b;
        }
    }
    return -1;
}

size_t mk_buf_bytes(int id) {
    return id >= 0 && id < kNumBufs ? g_state.t.bytes[id] : 0;
}

int mk_read(int id, void* host, size_t bytes) {
    if (!g_state.ready || id < 0 || id >= kNumBufs || bytes > g_state.t.bytes[id]) {
        return 1;
    }
    return cudaMemcpy(host, g_state.ws + g_state.t.off[id], bytes, cudaMemcpyDeviceToHost) != cudaSuccess;
}

// C[M][N] = A[M][K] · W[N][K]ᵀ through the tcgen05 engine with the plain f32 epilogue.
// tile = 64, 128 or 256 picks the column tile; anything else lets the library choose.
int mk_gemm_test(const uint16_t* A, const uint16_t* W, float* C, int M, int N, int K, int tile) {
    Device dev;
    if (device_state(dev)) {
        fprintf(stderr, "mk_gemm_test: %s\n", g_error.c_str());
        return 1;
    }
    if (M < 1 || N < 64 || N % 64 || K < kBK || K % kBK) {
        fprintf(stderr, "mk_gemm_test: N must be a multiple of 64 and K of %d\n", kBK);
        return 1;
    }
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(reinterpret_cast<const void*>(gemm_test_kernel), cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSmemAlloc);
        attr = true;
    }
    bf16 *da = nullptr, *dw = nullptr;
    float* dc = nullptr;
    Control* ctl = nullptr;
    const bool got = cudaMalloc(&da, size_t(M) * K * 2) == cudaSuccess && cudaMalloc(&dw, size_t(N) * K * 2) == cudaSuccess &&
                     cudaMalloc(&dc, size_t(M) * N * 4) == cudaSuccess && cudaMalloc(&ctl, sizeof(Control)) == cudaSuccess &&
                     cudaMemset(ctl, 0, sizeof(Control)) == cudaSuccess &&
                     cudaMemcpy(da, A, size_t(M) * K * 2, cudaMemcpyHostToDevice) == cudaSuccess &&
                     cudaMemcpy(dw, W, size_t(N) * K * 2, cudaMemcpyHostToDevice) == cudaSuccess;
    if (!got) { // nothing is launched on buffers that do not exist
        fprintf(stderr, "mk_gemm_test: device buffers: %s\n", cudaGetErrorString(cudaGetLastError()));
        cudaFree(da), cudaFree(dw), cudaFree(dc), cudaFree(ctl);
        return 1;
    }
    int bn = (tile == 64 || tile == 128 || tile == 256) && N % tile == 0 ? tile : choose_bn(M, N, dev.sms);
    Launch L;
    memset(&L, 0, sizeof L);
    L.kp.ctl = ctl, L.kp.wait_cycles = kWaitCycles;
    int rc = encode_map(&L.tmap[0], da, M, K, K, kBM) || encode_map(&L.tmap[1], dw, N, K, K, bn);
    if (!rc) {
        GemmDesc g{};
        g.map_a = 0, g.map_b = 1, g.m = M, g.n = N, g.k = K, g.bn = bn, g.epi = EPI_F32, g.out = dc, g.ldo = N, g.map_o = -1;
        g.sig_from = N, g.bias_cols = N, g.period = 1;
        const int tiles = cdiv(M, kBM) * (N / bn);
        gemm_test_kernel<<<tiles < dev.sms ? tiles : dev.sms, kThreads, kSmemAlloc>>>(L, g);
        rc = cudaDeviceSynchronize() != cudaSuccess;
        if (rc) {
            fprintf(stderr, "mk_gemm_test: %s\n", cudaGetErrorString(cudaGetLastError()));
        }
        Control c{};
        cudaMemcpy(&c, ctl, sizeof c, cudaMemcpyDeviceToHost);
        if (c.status != ST_OK) {
            fprintf(stderr, "mk_gemm_test: the kernel gave up waiting (status %u)\n", c.status);
            rc = 1;
        }
        cudaMemcpy(C, dc, size_t(M) * N * 4, cudaMemcpyDeviceToHost);
    } else {
        fprintf(stderr, "mk_gemm_test: %s\n", g_error.c_str());
    }
    cudaFree(da), cudaFree(dw), cudaFree(dc), cudaFree(ctl);
    return rc ? 1 : 0;
}

} // extern "C"
