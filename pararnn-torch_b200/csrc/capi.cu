// extern "C" entry points declared in include/pararnn_b200.h.  This file owns
// argument validation, the workspace layout and the sequence of launches that
// make up one fused forward or backward call; the kernels live in the other .cu files.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/pararnn_b200.h"
#include "kernels.h"

using namespace prb;

static_assert(sizeof(prb_stats) == sizeof(DeviceStats), "stats layout");
static_assert(PRB_MAX_ITERS == kMaxIters, "history capacity");

namespace {

// Bump allocator over the caller's workspace.  With base == nullptr it only
// measures, so the size query and the real layout cannot drift apart.
struct Bump {
    char* base;
    size_t off = 0;
    explicit Bump(void* b) : base(reinterpret_cast<char*>(b)) {}
    template <typename T>
    T* take(size_t n) {
        off = (off + 255) & ~size_t(255);
        T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
        off += n * sizeof(T);
        return p;
    }
};

constexpr int kTickets = 64;

struct ChainScratch {
    unsigned* flags;
    unsigned* tickets;
    float* agg;
    float* inc;
    int n_chains;
    int max_tt;
    unsigned next_epoch = 1;
    int next_ticket = 0;
};

// nv = floats per lane of the widest map that will travel on this chain
ChainScratch plan_chain(Bump& b, int B, int T, int d, int min_tile_steps, int nv) {
    ChainScratch c;
    c.n_chains = B * ((d + kLanes - 1) / kLanes);
    c.max_tt = (T + min_tile_steps - 1) / min_tile_steps;
    const size_t tiles = (size_t)c.n_chains * c.max_tt;
    c.flags = b.take<unsigned>(tiles + kTickets);
    c.tickets = c.flags ? c.flags + tiles : nullptr;
    c.agg = b.take<float>(tiles * nv * kLanes);
    c.inc = b.take<float>(tiles * nv * kLanes);
    return c;
}

Chain next_chain(ChainScratch& c, int T, int tile_steps, int* status) {
    Chain ch;
    ch.flags = c.flags;
    ch.agg = c.agg;
    ch.inc = c.inc;
    ch.ticket = c.tickets + (c.next_ticket++ % kTickets);
    ch.status = status;
    ch.epoch = c.next_epoch++;
    ch.spin_limit = options().spin_limit;
    ch.n_chains = c.n_chains;
    ch.n_tt = (T + tile_steps - 1) / tile_steps;
    return ch;
}

template <typename T>
__global__ void cvt_to_f32_kernel(const T* src, float* dst, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        dst[i] = ld_f(src + i);
}
template <typename T>
__global__ void cvt_from_f32_kernel(const float* src, T* dst, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        st_f(dst + i, src[i]);
}

void to_f32(const void* src, float* dst, size_t n, int dtype, cudaStream_t s) {
    const size_t cap = (size_t)sm_count() * 8;
    const int blocks = (int)((n + 255) / 256 < cap ? (n + 255) / 256 : cap);
    if (dtype == kF32)
        cvt_to_f32_kernel<float><<<blocks, 256, 0, s>>>((const float*)src, dst, n);
    else
        cvt_to_f32_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)src, dst, n);
}
void from_f32(const float* src, void* dst, size_t n, int dtype, cudaStream_t s) {
    const size_t cap = (size_t)sm_count() * 8;
    const int blocks = (int)((n + 255) / 256 < cap ? (n + 255) / 256 : cap);
    if (dtype == kF32)
        cvt_from_f32_kernel<float><<<blocks, 256, 0, s>>>(src, (float*)dst, n);
    else
        cvt_from_f32_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(src, (__nv_bfloat16*)dst, n);
}

// Kernel family for a sLSTM pass: 0 = look-back kernels (any shape), 2 = warp-pipelined
// persistent kernels (one CTA per chain, TMA-fed).  One CTA walks a whole chain, so the
// pipelined family needs a minimum of chains to win over the look-back kernels, which also split
// the time axis: measured cross-over at about 32 chains (B=1, T=65536, d=1024: 12.1 ms against
// 13.7 ms per forward + backward).  prb_debug_set(PRB_OPT_KERNEL_FAMILY) overrides the choice so
// that the tests can cover both families on small shapes.
constexpr int kMinChainsPersistent = 32;

int kernel_path(int dtype, int B, int T, int d) {
    const int forced = options().kernel_family;
    if (forced == 0) return 0;
    if (!tma_addressable(dtype, B, T, d)) return 0;
    if (forced == 2) return 2;
    return B * ((d + kLanes - 1) / kLanes) >= kMinChainsPersistent ? 2 : 0;
}
// aggregate-only sweeps: one CTA per chain when there are enough chains (or when the pipelined
// family is forced), else the look-back kernels with map carries
bool agg_seg(int B, int d) {
    const int forced = options().kernel_family;
    if (forced == 0) return false;
    if (forced == 2) return true;
    return B * ((d + kLanes - 1) / kLanes) >= kMinChainsPersistent;
}

// scalar-diagonal cells: pipelined persistent kernels when TMA can address the arrays and there
// are enough chains to occupy a good part of the GPU (one CTA per chain); else look-back kernels
bool diag_pipe(int dtype, int B, int T, int d) {
    const int forced = options().kernel_family;
    if (forced == 0) return false;
    if (!tma_addressable(dtype, B, T, d)) return false;
    if (forced == 2) return true;
    return B * ((d + kLanes - 1) / kLanes) >= 48;
}

bool bad_dtype(int dtype) { return dtype != kF32 && dtype != kBF16; }
bool misaligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 255u) != 0; }

int check_ws(void* ws, size_t have, size_t need) {
    if (need == 0) return PRB_OK;
    if (!ws || misaligned(ws) || have < need) return PRB_ERR_WORKSPACE;
    return PRB_OK;
}

// ---------------------------------------------------------------- diag cells
struct DiagPlan {
    ChainScratch chain;
    float* par;
    float* h0;
    float* buf[2];
    size_t total;
};

DiagPlan plan_diag_fwd(void* ws, int cell, int B, int T, int d, int K, bool has_h0) {
    Bump b(ws);
    DiagPlan p;
    const int np = diag_cell_params(cell);
    p.chain = plan_chain(b, B, T, d, diag_tile_steps(), 2);
    p.par = b.take<float>((size_t)np * d);
    p.h0 = b.take<float>((size_t)B * d);
    const size_t n = (size_t)B * T * d;
    p.buf[0] = K >= 2 ? b.take<float>(n) : nullptr;
    p.buf[1] = K >= 3 ? b.take<float>(n) : nullptr;
    (void)has_h0;
    p.total = b.off + 256;
    return p;
}

int run_diag_fwd(int cell, const void* wx, const void* const* pars, const void* h0, void* out, int B,
                 int T, int d, int dtype, int K, float omega, int want_residual, void* ws,
                 size_t ws_bytes, prb_stats* stats, cudaStream_t s) {
    if (!wx || !out || !stats || B < 1 || T < 1 || d < 1 || K < 0 || K > kMaxIters || bad_dtype(dtype))
        return PRB_ERR_BAD_ARG;
    const int np = diag_cell_params(cell);
    for (int i = 0; i < np; ++i)
        if (!pars[i]) return PRB_ERR_BAD_ARG;
    DiagPlan p = plan_diag_fwd(nullptr, cell, B, T, d, K, h0 != nullptr);
    if (int e = check_ws(ws, ws_bytes, p.total)) return e;
    p = plan_diag_fwd(ws, cell, B, T, d, K, h0 != nullptr);
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    cudaMemsetAsync(st, 0, sizeof(DeviceStats), s);
    cudaMemsetAsync(p.chain.flags, 0, ((size_t)p.chain.n_chains * p.chain.max_tt + kTickets) * 4, s);
    for (int i = 0; i < np; ++i) to_f32(pars[i], p.par + (size_t)i * d, d, dtype, s);
    const float* h0f = nullptr;
    if (h0) {
        to_f32(h0, p.h0, (size_t)B * d, dtype, s);
        h0f = p.h0;
    }
    if (K == 0) {
        launch_diag_guess(cell, dtype, false, wx, p.par, h0f, out, B, T, d, s);
    }
    bool fused_done = false;
    if (K >= 1 && options().newton_fused && diag_pipe(dtype, B, T, d)) {
        // all iterations in one sweep (no work trajectory); shapes it cannot take fall through
        DiagFwdArgs a{};
        a.wx = wx;
        a.par = p.par;
        a.halo = h0f;
        a.hout = out;
        a.resid_bits = &st->hist_bits[0];
        a.final_bits = want_residual ? &st->final_bits : nullptr;
        a.B = B;
        a.T = T;
        a.d = d;
        a.omega = omega;
        a.chain = next_chain(p.chain, T, diag_tile_steps(), &st->status);
        const cudaError_t e = launch_diag_newton_fused(cell, dtype, a, K, s);
        if (e == cudaSuccess)
            fused_done = true;
        else if (e != cudaErrorNotSupported)
            return PRB_ERR_LAUNCH;
    }
    for (int k = 0; k < K && !fused_done; ++k) {
        DiagFwdArgs a{};
        a.wx = wx;
        a.par = p.par;
        a.halo = h0f;
        a.carry_in = nullptr;
        a.hin = k > 0 ? p.buf[(k - 1) & 1] : nullptr;
        a.hout = (k == K - 1) ? out : (void*)p.buf[k & 1];
        a.resid_bits = &st->hist_bits[k];
        a.final_bits = (want_residual && k == K - 1) ? &st->final_bits : nullptr;
        a.B = B;
        a.T = T;
        a.d = d;
        a.omega = omega;
        a.chain = next_chain(p.chain, T, diag_tile_steps(), &st->status);
        cudaError_t e = cudaErrorNotSupported;
        if (diag_pipe(dtype, B, T, d)) e = launch_diag_newton_pipe(cell, dtype, a, k == 0, k == K - 1, s);
        if (e == cudaErrorNotSupported) e = launch_diag_newton(cell, dtype, a, k == 0, k == K - 1, s);
        if (e != cudaSuccess) return PRB_ERR_LAUNCH;
    }
    if (want_residual && K == 0)
        if (launch_diag_residual(cell, dtype, false, wx, p.par, h0f, out, B, T, d, &st->final_bits, s) !=
            cudaSuccess)
            return PRB_ERR_LAUNCH;
    return cudaGetLastError() == cudaSuccess ? PRB_OK : PRB_ERR_LAUNCH;
}

struct DiagBwdPlan {
    ChainScratch chain;
    float* par;
    float* h0;
    float* partial;
    size_t total;
};

DiagBwdPlan plan_diag_bwd(void* ws, int cell, int B, int T, int d) {
    Bump b(ws);
    DiagBwdPlan p;
    const int np = diag_cell_params(cell);
    p.chain = plan_chain(b, B, T, d, diag_tile_steps(), 2);
    p.par = b.take<float>((size_t)np * d);
    p.h0 = b.take<float>((size_t)B * d);
    // parameter rows, then the per-gate bias rows
    p.partial = b.take<float>((size_t)B * p.chain.max_tt * (np + diag_cell_gates(cell)) * d);
    p.total = b.off + 256;
    return p;
}

int run_diag_bwd(int cell, const void* states, const void* wx, const void* const* pars,
                 const void* h0, const void* grad_states, void* g_wx, float* g_params, float* g_h0,
                 int B, int T, int d, int dtype, void* ws, size_t ws_bytes, prb_stats* stats,
                 cudaStream_t s, float* g_bias = nullptr) {
    if (!states || !wx || !grad_states || !g_wx || !g_params || !stats || B < 1 || T < 1 || d < 1 ||
        bad_dtype(dtype))
        return PRB_ERR_BAD_ARG;
    const int np = diag_cell_params(cell);
    for (int i = 0; i < np; ++i)
        if (!pars[i]) return PRB_ERR_BAD_ARG;
    DiagBwdPlan p = plan_diag_bwd(nullptr, cell, B, T, d);
    if (int e = check_ws(ws, ws_bytes, p.total)) return e;
    p = plan_diag_bwd(ws, cell, B, T, d);
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    cudaMemsetAsync(st, 0, sizeof(DeviceStats), s);
    cudaMemsetAsync(p.chain.flags, 0, ((size_t)p.chain.n_chains * p.chain.max_tt + kTickets) * 4, s);
    for (int i = 0; i < np; ++i) to_f32(pars[i], p.par + (size_t)i * d, d, dtype, s);
    const float* h0f = nullptr;
    if (h0) {
        to_f32(h0, p.h0, (size_t)B * d, dtype, s);
        h0f = p.h0;
    }
    DiagBwdArgs a{};
    a.wx = wx;
    a.states = states;
    a.grad_states = grad_states;
    a.par = p.par;
    a.halo = h0f;
    a.g_wx = g_wx;
    a.gp_partial = p.partial;
    a.gb_partial = g_bias ? p.partial + (size_t)B * p.chain.max_tt * np * d : nullptr;
    a.g_h0 = g_h0;
    a.B = B;
    a.T = T;
    a.d = d;
    a.chain = next_chain(p.chain, T, diag_tile_steps(), &st->status);
    bool pipe = diag_pipe(dtype, B, T, d);
    cudaError_t e = cudaErrorNotSupported;
    if (pipe) e = launch_diag_bwd_pipe(cell, dtype, a, s);
    if (e == cudaErrorNotSupported) {
        pipe = false;
        e = launch_diag_bwd(cell, dtype, a, false, s);
    }
    if (e != cudaSuccess) return PRB_ERR_LAUNCH;
    // one partial row per tile (look-back) or per batch row (one CTA per chain)
    const int rows = pipe ? B : B * a.chain.n_tt;
    if (launch_reduce_partials(p.partial, rows, np * d, g_params, s) != cudaSuccess) return PRB_ERR_LAUNCH;
    if (g_bias && launch_reduce_partials(a.gb_partial, rows, diag_cell_gates(cell) * d, g_bias, s) != cudaSuccess)
        return PRB_ERR_LAUNCH;
    return PRB_OK;
}

// ---------------------------------------------------------------- sLSTM
struct SlstmPlan {
    ChainScratch chain;
    float* r;
    float* h0;
    float* hb[2];
    float* sb[2];
    size_t total;
};

SlstmPlan plan_slstm_fwd(void* ws, int B, int T, int d, int K, int P, bool has_guess) {
    Bump b(ws);
    SlstmPlan p;
    const int min_tile = slstm_tile_steps() < slstm_picard_tile_steps() ? slstm_tile_steps()
                                                                         : slstm_picard_tile_steps();
    p.chain = plan_chain(b, B, T, d, min_tile, 20);
    p.r = b.take<float>((size_t)4 * d);
    p.h0 = b.take<float>((size_t)B * 4 * d);
    const size_t nh = (size_t)B * T * d;
    const bool picard = !has_guess;
    p.hb[0] = (picard && P >= 1) ? b.take<float>(nh) : nullptr;
    p.hb[1] = (picard && P >= 2) ? b.take<float>(nh) : nullptr;
    p.sb[0] = b.take<float>(nh * 4);
    p.sb[1] = K >= 2 ? b.take<float>(nh * 4) : nullptr;
    p.total = b.off + 256;
    return p;
}

int run_slstm_fwd(const void* wx, const void* r, const void* h0, const void* guess, void* out, int B,
                  int T, int d, int dtype, int K, int P, float omega, float eps, int want_residual,
                  void* ws, size_t ws_bytes, prb_stats* stats, cudaStream_t s) {
    // every pass of the look-back family takes its own ticket counter
    if (!wx || !r || !out || !stats || B < 1 || T < 1 || d < 1 || K < 0 || K > kMaxIters || P < 0 ||
        P + 1 + K > kTickets || bad_dtype(dtype))
        return PRB_ERR_BAD_ARG;
    SlstmPlan p = plan_slstm_fwd(nullptr, B, T, d, K, P, guess != nullptr);
    if (int e = check_ws(ws, ws_bytes, p.total)) return e;
    p = plan_slstm_fwd(ws, B, T, d, K, P, guess != nullptr);
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    cudaMemsetAsync(st, 0, sizeof(DeviceStats), s);
    cudaMemsetAsync(p.chain.flags, 0, ((size_t)p.chain.n_chains * p.chain.max_tt + kTickets) * 4, s);
    to_f32(r, p.r, (size_t)4 * d, dtype, s);
    const float* h0f = nullptr;
    if (h0) {
        to_f32(h0, p.h0, (size_t)B * 4 * d, dtype, s);
        h0f = p.h0;
    }
    const size_t nst = (size_t)B * T * 4 * d;
    const int path = kernel_path(dtype, B, T, d);
    if (guess) {
        to_f32(guess, p.sb[0], nst, dtype, s);
    } else {
        // the pipelined family runs all P+1 passes in one sweep when it can
        bool fused_done = false;
        if (path == 2 && P + 1 <= slstm_picard_fused_max_passes() && options().picard_fused) {
            SlstmPicardArgs a{};
            a.wx = wx;
            a.r = p.r;
            a.h_halo = h0f ? h0f + 3 * (size_t)d : nullptr;
            a.halo_stride = 4 * d;
            a.carry_in = h0f;
            a.carry_stride = 4 * d;
            a.state_out = p.sb[0];
            a.B = B;
            a.T = T;
            a.d = d;
            a.eps = eps;
            a.chain = next_chain(p.chain, T, slstm_picard_tile_steps(), &st->status);
            const cudaError_t e = launch_slstm_picard_fused(dtype, a, P + 1, s);
            if (e == cudaSuccess) fused_done = true;
            else if (e != cudaErrorNotSupported) return PRB_ERR_LAUNCH;
        }
        for (int pass = 0; pass <= P && !fused_done; ++pass) {
            SlstmPicardArgs a{};
            a.wx = wx;
            a.r = p.r;
            a.h_prev = pass > 0 ? p.hb[(pass - 1) & 1] : nullptr;
            a.h_halo = h0f ? h0f + 3 * (size_t)d : nullptr;
            a.halo_stride = 4 * d;
            a.carry_in = h0f;  // slots (c, n, m) of h0
            a.carry_stride = 4 * d;
            if (pass == P)
                a.state_out = p.sb[0];
            else
                a.h_out = p.hb[pass & 1];
            a.B = B;
            a.T = T;
            a.d = d;
            a.eps = eps;
            a.chain = next_chain(p.chain, T, slstm_picard_tile_steps(), &st->status);
            cudaError_t e = cudaErrorNotSupported;
            if (path == 2) e = launch_slstm_picard_pipe(dtype, a, s);
            if (e == cudaErrorNotSupported) e = launch_slstm_picard(dtype, a, false, s);
            if (e != cudaSuccess) return PRB_ERR_LAUNCH;
        }
    }
    if (K == 0) from_f32(p.sb[0], out, nst, dtype, s);
    // the pipelined family runs all K iterations in one sweep when it can
    bool newton_done = false;
    if (path == 2 && K >= 1 && K <= slstm_newton_fused_max_iters() && options().newton_fused) {
        SlstmNewtonArgs a{};
        a.wx = wx;
        a.r = p.r;
        a.sin = p.sb[0];
        a.halo = h0f;
        a.halo_stride = 4 * d;
        a.sout = out;
        a.resid_bits = &st->hist_bits[0];
        a.final_bits = want_residual ? &st->final_bits : nullptr;
        a.B = B;
        a.T = T;
        a.d = d;
        a.omega = omega;
        a.eps = eps;
        a.chain = next_chain(p.chain, T, slstm_tile_steps(), &st->status);
        const cudaError_t e = launch_slstm_newton_fused(dtype, a, K, s);
        if (e == cudaSuccess) newton_done = true;
        else if (e != cudaErrorNotSupported) return PRB_ERR_LAUNCH;
    }
    for (int k = 0; k < K && !newton_done; ++k) {
        SlstmNewtonArgs a{};
        a.wx = wx;
        a.r = p.r;
        a.sin = p.sb[k & 1];
        a.halo = h0f;
        a.halo_stride = 4 * d;
        a.sout = (k == K - 1) ? out : (void*)p.sb[(k + 1) & 1];
        a.resid_bits = &st->hist_bits[k];
        a.final_bits = (want_residual && k == K - 1) ? &st->final_bits : nullptr;
        a.B = B;
        a.T = T;
        a.d = d;
        a.omega = omega;
        a.eps = eps;
        a.chain = next_chain(p.chain, T, slstm_tile_steps(), &st->status);
        cudaError_t e = cudaErrorNotSupported;
        if (path == 2) e = launch_slstm_newton_pipe(dtype, a, k == K - 1, s);
        if (e == cudaErrorNotSupported) e = launch_slstm_newton(dtype, a, k == K - 1, false, s);
        if (e != cudaSuccess) return PRB_ERR_LAUNCH;
    }
    if (want_residual && K == 0)
        if (launch_slstm_residual(dtype, false, wx, p.r, h0f, 4 * d, out, B, T, d, eps, &st->final_bits,
                                  s) != cudaSuccess)
            return PRB_ERR_LAUNCH;
    return cudaGetLastError() == cudaSuccess ? PRB_OK : PRB_ERR_LAUNCH;
}

struct SlstmBwdPlan {
    ChainScratch chain;
    float* r;
    float* h0;
    float* partial;
    size_t total;
};

SlstmBwdPlan plan_slstm_bwd(void* ws, int B, int T, int d) {
    Bump b(ws);
    SlstmBwdPlan p;
    p.chain = plan_chain(b, B, T, d, slstm_tile_steps(), 20);
    p.r = b.take<float>((size_t)4 * d);
    p.h0 = b.take<float>((size_t)B * 4 * d);
    p.partial = b.take<float>((size_t)B * p.chain.max_tt * 8 * d);  // grad R rows, then bias rows
    p.total = b.off + 256;
    return p;
}


// Carry entering a rank of a time-sharded pass.  `gathered` holds one slot per rank
// (slot stride nv*B*d floats): the first rank in scan order stores the exact carry leaving it
// (ns floats per channel), every other rank its shard aggregate map (nv floats per channel).
// carry(rank) = map(rank-1) o ... o map(first+1) applied to tail(first).
template <class M>
__global__ void fold_carries_kernel(const float* gathered, int rank, int world, int reverse, float* out,
                                    int B, int d, int nv_slot) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * d) return;
    const int b = idx / d, ch = idx % d;
    const size_t slot = (size_t)nv_slot * B * d;
    const int first = reverse ? world - 1 : 0;
    const int step = reverse ? -1 : 1;
    float vec[M::NS];
    const float* p0 = gathered + (size_t)first * slot + (size_t)b * nv_slot * d + ch;
#pragma unroll
    for (int i = 0; i < M::NS; ++i) vec[i] = p0[(size_t)i * d];
    for (int q = first + step; q != rank; q += step) {
        float m[M::NV];
        const float* p = gathered + (size_t)q * slot + (size_t)b * nv_slot * d + ch;
#pragma unroll
        for (int i = 0; i < M::NV; ++i) m[i] = p[(size_t)i * d];
        M::apply(m, vec);
    }
#pragma unroll
    for (int i = 0; i < M::NS; ++i) out[((size_t)b * M::NS + i) * d + ch] = vec[i];
}

// Carries entering the time segments of one rank (segments in time order; the scan runs through
// them forwards, or backwards when reverse != 0).  out[j] (j < n_seg) is the carry entering
// segment j, out[n_seg] the carry leaving the rank.  carry0 == nullptr means a zero carry.
template <class M>
__global__ void segment_carries_kernel(const float* agg, int n_seg, int reverse, const float* carry0,
                                       float* out, int B, int d) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * d) return;
    const int b = idx / d, ch = idx % d;
    float vec[M::NS];
#pragma unroll
    for (int i = 0; i < M::NS; ++i) vec[i] = carry0 ? carry0[((size_t)b * M::NS + i) * d + ch] : 0.f;
    for (int k = 0; k < n_seg; ++k) {
        const int j = reverse ? n_seg - 1 - k : k;
#pragma unroll
        for (int i = 0; i < M::NS; ++i) out[(((size_t)j * B + b) * M::NS + i) * d + ch] = vec[i];
        float m[M::NV];
        const float* p = agg + ((size_t)j * B + b) * M::NV * d + ch;
#pragma unroll
        for (int i = 0; i < M::NV; ++i) m[i] = p[(size_t)i * d];
        M::apply(m, vec);
    }
#pragma unroll
    for (int i = 0; i < M::NS; ++i) out[(((size_t)n_seg * B + b) * M::NS + i) * d + ch] = vec[i];
}

// fold_carries_kernel and segment_carries_kernel in one launch, for a rank that is not the first in
// scan order: the carry entering the rank is folded from the gathered slots (slot stride slot_rows
// floats per channel: the map or tail in the first rows, anything riding along after them), written
// to carry_out and pushed through the rank's own segment maps.  For the frozen-gate passes the
// hidden value at the previous rank's last step follows from the carry and that step's output-gate
// pre-activation, which the previous rank ships in row NV of its slot: h_end = sigmoid(zo) c / (n + eps).
template <class M>
__global__ void shard_carries_kernel(const float* gathered, int slot_rows, int rank, int world, int reverse,
                                     const float* agg, int n_seg, float* carry_out, float* carries, float eps,
                                     float* h_end, int B, int d) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * d) return;
    const int b = idx / d, ch = idx % d;
    const size_t slot = (size_t)slot_rows * B * d;
    const int first = reverse ? world - 1 : 0;
    const int step = reverse ? -1 : 1;
    float vec[M::NS];
    const float* p0 = gathered + (size_t)first * slot + (size_t)b * slot_rows * d + ch;
#pragma unroll
    for (int i = 0; i < M::NS; ++i) vec[i] = p0[(size_t)i * d];
    for (int q = first + step; q != rank; q += step) {
        float m[M::NV];
        const float* p = gathered + (size_t)q * slot + (size_t)b * slot_rows * d + ch;
#pragma unroll
        for (int i = 0; i < M::NV; ++i) m[i] = p[(size_t)i * d];
        M::apply(m, vec);
    }
#pragma unroll
    for (int i = 0; i < M::NS; ++i) carry_out[((size_t)b * M::NS + i) * d + ch] = vec[i];
    if (h_end) {
        const float zo = gathered[(size_t)(rank - step) * slot + ((size_t)b * slot_rows + M::NV) * d + ch];
        h_end[(size_t)b * d + ch] = sigmoid_f(zo) * vec[0] / (vec[1] + eps);
    }
    if (!carries) return;
    for (int k = 0; k < n_seg; ++k) {
        const int j = reverse ? n_seg - 1 - k : k;
#pragma unroll
        for (int i = 0; i < M::NS; ++i) carries[(((size_t)j * B + b) * M::NS + i) * d + ch] = vec[i];
        float m[M::NV];
        const float* p = agg + ((size_t)j * B + b) * M::NV * d + ch;
#pragma unroll
        for (int i = 0; i < M::NV; ++i) m[i] = p[(size_t)i * d];
        M::apply(m, vec);
    }
#pragma unroll
    for (int i = 0; i < M::NS; ++i) carries[(((size_t)n_seg * B + b) * M::NS + i) * d + ch] = vec[i];
}

// Map of a whole rank = composition of its segment maps in scan order.
template <class M>
__global__ void fold_segments_kernel(const float* agg, int n_seg, int reverse, float* out, int B, int d) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * d) return;
    const int b = idx / d, ch = idx % d;
    float acc[M::NV];
    for (int k = 0; k < n_seg; ++k) {
        const int j = reverse ? n_seg - 1 - k : k;
        float m[M::NV];
        const float* p = agg + ((size_t)j * B + b) * M::NV * d + ch;
#pragma unroll
        for (int i = 0; i < M::NV; ++i) m[i] = p[(size_t)i * d];
        if (k == 0) {
#pragma unroll
            for (int i = 0; i < M::NV; ++i) acc[i] = m[i];
        } else {
            M::compose(acc, m);
        }
    }
#pragma unroll
    for (int i = 0; i < M::NV; ++i) out[((size_t)b * M::NV + i) * d + ch] = acc[i];
}

// Segments must tile [0, T) exactly once, and there may be no more of them than time tiles of the
// look-back kernels: the per-pass workspace holds one parameter-partial row per tile.
bool bad_segments(int T, int n_seg, int seg_len) {
    if (n_seg < 1 || seg_len < 1) return true;
    if (n_seg == 1) return false;
    const int tile = slstm_tile_steps() < slstm_picard_tile_steps() ? slstm_tile_steps() : slstm_picard_tile_steps();
    if (n_seg > (T + tile - 1) / tile) return true;
    return (long long)(n_seg - 1) * seg_len >= T || (long long)n_seg * seg_len < T;
}

}  // namespace

extern "C" {

const char* prb_version(void) { return "pararnn_b200 0.2 (sm_100a)"; }

int prb_debug_set(int option, long long value) {
    Options& o = options();
    switch (option) {
        case PRB_OPT_KERNEL_FAMILY:
            if (value != -1 && value != 0 && value != 2) return PRB_ERR_BAD_ARG;
            o.kernel_family = (int)value;
            return PRB_OK;
        case PRB_OPT_PICARD_FUSED: o.picard_fused = value != 0; return PRB_OK;
        case PRB_OPT_NEWTON_FUSED: o.newton_fused = value != 0; return PRB_OK;
        case PRB_OPT_SPIN_LIMIT:
            o.spin_limit = value <= 0 ? kSpinLimit : (unsigned)(value > 0x7fffffffLL ? 0x7fffffffLL : value);
            return PRB_OK;
        default: return PRB_ERR_BAD_ARG;
    }
}

const char* prb_error_string(int code) {
    switch (code) {
        case PRB_OK: return "ok";
        case PRB_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or unknown enum)";
        case PRB_ERR_WORKSPACE: return "workspace missing, not 256-byte aligned, or too small";
        case PRB_ERR_UNSUPPORTED: return "shape not supported by this kernel";
        case PRB_ERR_LAUNCH: return "CUDA launch error";
        case PRB_ERR_TOO_LARGE: return "size exceeds the fixed capacity of this entry point";
        case PRB_STATUS_CHAIN_TIMEOUT: return "a bounded device-side wait ran out";
        default: return "unknown code";
    }
}

size_t prb_newton_workspace_bytes(int cell, int dtype, int B, int T, int d, int n_heads,
                                  int max_iters, int picard_iters) {
    (void)dtype;
    (void)n_heads;
    if (B < 1 || T < 1 || d < 1) return 0;
    if (is_diag_cell(cell)) return plan_diag_fwd(nullptr, cell, B, T, d, max_iters, true).total;
    if (cell == kCellSlstmDiag) return plan_slstm_fwd(nullptr, B, T, d, max_iters, picard_iters, false).total;
    return 0;
}

size_t prb_bwd_workspace_bytes(int cell, int dtype, int B, int T, int d, int n_heads) {
    (void)dtype;
    (void)n_heads;
    if (B < 1 || T < 1 || d < 1) return 0;
    if (is_diag_cell(cell)) return plan_diag_bwd(nullptr, cell, B, T, d).total;
    if (cell == kCellSlstmDiag) return plan_slstm_bwd(nullptr, B, T, d).total;
    return 0;
}

int prb_newton_gru_fused(const void* wx, const void* a_z, const void* a_r, const void* a_n,
                         const void* h0, void* out, int B, int T, int d, int dtype, int max_iters,
                         float omega, int want_residual, void* workspace, size_t workspace_bytes,
                         prb_stats* stats, prb_stream_t stream) {
    const void* pars[3] = {a_z, a_r, a_n};
    return run_diag_fwd(kCellGruDiag, wx, pars, h0, out, B, T, d, dtype, max_iters, omega,
                        want_residual, workspace, workspace_bytes, stats, (cudaStream_t)stream);
}

int prb_newton_nlru_fused(const void* wx, const void* u, const void* h0, void* out, int B, int T,
                          int d, int dtype, int max_iters, float omega, int want_residual,
                          void* workspace, size_t workspace_bytes, prb_stats* stats,
                          prb_stream_t stream) {
    const void* pars[3] = {u, nullptr, nullptr};
    return run_diag_fwd(kCellNlru, wx, pars, h0, out, B, T, d, dtype, max_iters, omega, want_residual,
                        workspace, workspace_bytes, stats, (cudaStream_t)stream);
}

int prb_newton_titans_fused(const void* wx, const void* u, const void* r, const void* h0, void* out, int B,
                            int T, int d, int dtype, int max_iters, float omega, int want_residual,
                            void* workspace, size_t workspace_bytes, prb_stats* stats, prb_stream_t stream) {
    const void* pars[3] = {u, r, nullptr};
    return run_diag_fwd(kCellTitans, wx, pars, h0, out, B, T, d, dtype, max_iters, omega, want_residual,
                        workspace, workspace_bytes, stats, (cudaStream_t)stream);
}

int prb_bwd_titans(const void* states, const void* wx, const void* u, const void* r, const void* h0,
                   const void* grad_states, void* g_wx, float* g_params, float* g_h0, int B, int T, int d,
                   int dtype, void* workspace, size_t workspace_bytes, prb_stats* stats,
                   prb_stream_t stream) {
    const void* pars[3] = {u, r, nullptr};
    return run_diag_bwd(kCellTitans, states, wx, pars, h0, grad_states, g_wx, g_params, g_h0, B, T, d,
                        dtype, workspace, workspace_bytes, stats, (cudaStream_t)stream);
}

int prb_newton_cfc_fused(const void* wx, const void* u, const void* h0, void* out, int B, int T, int d,
                         int dtype, int max_iters, float omega, int want_residual, void* workspace,
                         size_t workspace_bytes, prb_stats* stats, prb_stream_t stream) {
    const void* pars[3] = {u, nullptr, nullptr};
    return run_diag_fwd(kCellCfc, wx, pars, h0, out, B, T, d, dtype, max_iters, omega, want_residual,
                        workspace, workspace_bytes, stats, (cudaStream_t)stream);
}

int prb_bwd_cfc(const void* states, const void* wx, const void* u, const void* h0, const void* grad_states,
                void* g_wx, float* g_params, float* g_h0, int B, int T, int d, int dtype, void* workspace,
                size_t workspace_bytes, prb_stats* stats, prb_stream_t stream) {
    const void* pars[3] = {u, nullptr, nullptr};
    return run_diag_bwd(kCellCfc, states, wx, pars, h0, grad_states, g_wx, g_params, g_h0, B, T, d, dtype,
                        workspace, workspace_bytes, stats, (cudaStream_t)stream);
}

int prb_bwd_diag_ex(int cell, const void* states, const void* wx, const void* p0, const void* p1,
                    const void* p2, const void* h0, const void* grad_states, void* g_wx, float* g_params,
                    float* g_bias, float* g_h0, int B, int T, int d, int dtype, void* workspace,
                    size_t workspace_bytes, prb_stats* stats, prb_stream_t stream) {
    if (!is_diag_cell(cell)) return PRB_ERR_BAD_ARG;
    const void* pars[3] = {p0, p1, p2};
    return run_diag_bwd(cell, states, wx, pars, h0, grad_states, g_wx, g_params, g_h0, B, T, d, dtype,
                        workspace, workspace_bytes, stats, (cudaStream_t)stream, g_bias);
}

/* ---- ParaLSTM --------------------------------------------------------------------------- */

namespace {
struct LstmPlan {
    ChainScratch chain;
    float* par;
    float* h0;
    float* buf[2];
    float* partial;
    size_t total;
};
LstmPlan plan_lstm(void* ws, int B, int T, int d, int K, bool bwd) {
    Bump b(ws);
    LstmPlan p;
    p.chain = plan_chain(b, B, T, d, lstm_tile_steps(), 6);
    p.par = b.take<float>((size_t)5 * d);
    p.h0 = b.take<float>((size_t)B * 2 * d);
    const size_t n = (size_t)B * T * 2 * d;
    p.buf[0] = (!bwd && K >= 2) ? b.take<float>(n) : nullptr;
    p.buf[1] = (!bwd && K >= 3) ? b.take<float>(n) : nullptr;
    p.partial = bwd ? b.take<float>((size_t)B * p.chain.max_tt * 5 * d) : nullptr;
    p.total = b.off + 256;
    return p;
}
}  // namespace

size_t prb_lstm_workspace_bytes(int B, int T, int d, int max_iters, int backward) {
    if (B < 1 || T < 1 || d < 1) return 0;
    return plan_lstm(nullptr, B, T, d, max_iters, backward != 0).total;
}

int prb_newton_lstm_fused(const void* wx, const void* a_f, const void* a_z, const void* a_o, const void* c_f,
                          const void* c_o, const void* h0, void* out, int B, int T, int d, int dtype,
                          int max_iters, float omega, int want_residual, void* workspace,
                          size_t workspace_bytes, prb_stats* stats, prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    const int K = max_iters;
    if (!wx || !a_f || !a_z || !a_o || !c_f || !c_o || !out || !stats || B < 1 || T < 1 || d < 1 || K < 0 ||
        K > kMaxIters || bad_dtype(dtype))
        return PRB_ERR_BAD_ARG;
    LstmPlan p = plan_lstm(nullptr, B, T, d, K, false);
    if (int e = check_ws(workspace, workspace_bytes, p.total)) return e;
    p = plan_lstm(workspace, B, T, d, K, false);
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    cudaMemsetAsync(st, 0, sizeof(DeviceStats), s);
    cudaMemsetAsync(p.chain.flags, 0, ((size_t)p.chain.n_chains * p.chain.max_tt + kTickets) * 4, s);
    const void* pars[5] = {a_f, a_z, a_o, c_f, c_o};
    for (int i = 0; i < 5; ++i) to_f32(pars[i], p.par + (size_t)i * d, d, dtype, s);
    const float* h0f = nullptr;
    if (h0) {
        to_f32(h0, p.h0, (size_t)B * 2 * d, dtype, s);
        h0f = p.h0;
    }
    if (K == 0) {
        if (launch_lstm_guess(dtype, wx, p.par, h0f, out, B, T, d, s) != cudaSuccess) return PRB_ERR_LAUNCH;
        if (want_residual &&
            launch_lstm_residual(dtype, wx, p.par, h0f, out, B, T, d, &st->final_bits, s) != cudaSuccess)
            return PRB_ERR_LAUNCH;
        return PRB_OK;
    }
    if (options().newton_fused && diag_pipe(dtype, B, T, d)) {
        // all iterations in one sweep (no work trajectory); shapes it cannot take fall through
        LstmFwdArgs a{};
        a.wx = wx;
        a.par = p.par;
        a.halo = h0f;
        a.sout = out;
        a.resid_bits = &st->hist_bits[0];
        a.final_bits = want_residual ? &st->final_bits : nullptr;
        a.B = B;
        a.T = T;
        a.d = d;
        a.omega = omega;
        a.chain = next_chain(p.chain, T, lstm_tile_steps(), &st->status);
        const cudaError_t e = launch_lstm_newton_fused(dtype, a, K, s);
        if (e == cudaSuccess) return PRB_OK;
        if (e != cudaErrorNotSupported) return PRB_ERR_LAUNCH;
    }
    for (int k = 0; k < K; ++k) {
        LstmFwdArgs a{};
        a.wx = wx;
        a.par = p.par;
        a.halo = h0f;
        a.sin = k > 0 ? p.buf[(k - 1) & 1] : nullptr;
        a.sout = (k == K - 1) ? out : (void*)p.buf[k & 1];
        a.resid_bits = &st->hist_bits[k];
        a.final_bits = (want_residual && k == K - 1) ? &st->final_bits : nullptr;
        a.B = B;
        a.T = T;
        a.d = d;
        a.omega = omega;
        a.chain = next_chain(p.chain, T, lstm_tile_steps(), &st->status);
        if (launch_lstm_newton(dtype, a, k == 0, k == K - 1, s) != cudaSuccess) return PRB_ERR_LAUNCH;
    }
    return PRB_OK;
}

int prb_bwd_lstm(const void* states, const void* wx, const void* a_f, const void* a_z, const void* a_o,
                 const void* c_f, const void* c_o, const void* h0, const void* grad_states, void* g_wx,
                 float* g_params, float* g_h0, int B, int T, int d, int dtype, void* workspace,
                 size_t workspace_bytes, prb_stats* stats, prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!states || !wx || !a_f || !a_z || !a_o || !c_f || !c_o || !grad_states || !g_wx || !g_params || !stats ||
        B < 1 || T < 1 || d < 1 || bad_dtype(dtype))
        return PRB_ERR_BAD_ARG;
    LstmPlan p = plan_lstm(nullptr, B, T, d, 0, true);
    if (int e = check_ws(workspace, workspace_bytes, p.total)) return e;
    p = plan_lstm(workspace, B, T, d, 0, true);
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    cudaMemsetAsync(st, 0, sizeof(DeviceStats), s);
    cudaMemsetAsync(p.chain.flags, 0, ((size_t)p.chain.n_chains * p.chain.max_tt + kTickets) * 4, s);
    const void* pars[5] = {a_f, a_z, a_o, c_f, c_o};
    for (int i = 0; i < 5; ++i) to_f32(pars[i], p.par + (size_t)i * d, d, dtype, s);
    const float* h0f = nullptr;
    if (h0) {
        to_f32(h0, p.h0, (size_t)B * 2 * d, dtype, s);
        h0f = p.h0;
    }
    LstmBwdArgs a{};
    a.wx = wx;
    a.states = states;
    a.grad_states = grad_states;
    a.par = p.par;
    a.halo = h0f;
    a.g_wx = g_wx;
    a.gp_partial = p.partial;
    a.g_h0 = g_h0;
    a.B = B;
    a.T = T;
    a.d = d;
    a.chain = next_chain(p.chain, T, lstm_tile_steps(), &st->status);
    cudaError_t e = cudaErrorNotSupported;
    int rows = B * a.chain.n_tt;
    if (diag_pipe(dtype, B, T, d)) e = launch_lstm_bwd_pipe(dtype, a, s);
    if (e == cudaSuccess)
        rows = B;  // the pipelined kernel writes one partial row per batch row
    else if (e == cudaErrorNotSupported)
        e = launch_lstm_bwd(dtype, a, s);
    if (e != cudaSuccess) return PRB_ERR_LAUNCH;
    return launch_reduce_partials(p.partial, rows, 5 * d, g_params, s) == cudaSuccess ? PRB_OK : PRB_ERR_LAUNCH;
}

int prb_newton_slstm_fused(const void* wx, const void* r, const void* h0, const void* states_guess,
                           void* out, int B, int T, int d, int dtype, int max_iters,
                           int picard_iters, float omega, float eps, int want_residual,
                           void* workspace, size_t workspace_bytes, prb_stats* stats,
                           prb_stream_t stream) {
    return run_slstm_fwd(wx, r, h0, states_guess, out, B, T, d, dtype, max_iters, picard_iters, omega,
                         eps, want_residual, workspace, workspace_bytes, stats, (cudaStream_t)stream);
}

int prb_bwd_gru(const void* states, const void* wx, const void* a_z, const void* a_r,
                const void* a_n, const void* h0, const void* grad_states, void* g_wx,
                float* g_params, float* g_h0, int B, int T, int d, int dtype, void* workspace,
                size_t workspace_bytes, prb_stats* stats, prb_stream_t stream) {
    const void* pars[3] = {a_z, a_r, a_n};
    return run_diag_bwd(kCellGruDiag, states, wx, pars, h0, grad_states, g_wx, g_params, g_h0, B, T, d,
                        dtype, workspace, workspace_bytes, stats, (cudaStream_t)stream);
}

int prb_bwd_nlru(const void* states, const void* wx, const void* u, const void* h0,
                 const void* grad_states, void* g_wx, float* g_params, float* g_h0, int B, int T,
                 int d, int dtype, void* workspace, size_t workspace_bytes, prb_stats* stats,
                 prb_stream_t stream) {
    const void* pars[3] = {u, nullptr, nullptr};
    return run_diag_bwd(kCellNlru, states, wx, pars, h0, grad_states, g_wx, g_params, g_h0, B, T, d,
                        dtype, workspace, workspace_bytes, stats, (cudaStream_t)stream);
}

int prb_bwd_slstm_ex(const void* states, const void* wx, const void* r, const void* h0,
                     const void* grad, int grad_slot, void* g_wx, float* g_params, float* g_bias,
                     float* g_h0, int B, int T, int d, int dtype, float eps, void* workspace,
                     size_t workspace_bytes, prb_stats* stats, prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!states || !wx || !r || !grad || !g_wx || !g_params || !stats || B < 1 || T < 1 || d < 1 ||
        bad_dtype(dtype) || grad_slot < -1 || grad_slot > 3)
        return PRB_ERR_BAD_ARG;
    SlstmBwdPlan p = plan_slstm_bwd(nullptr, B, T, d);
    if (int e = check_ws(workspace, workspace_bytes, p.total)) return e;
    p = plan_slstm_bwd(workspace, B, T, d);
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    cudaMemsetAsync(st, 0, sizeof(DeviceStats), s);
    cudaMemsetAsync(p.chain.flags, 0, ((size_t)p.chain.n_chains * p.chain.max_tt + kTickets) * 4, s);
    to_f32(r, p.r, (size_t)4 * d, dtype, s);
    const float* h0f = nullptr;
    if (h0) {
        to_f32(h0, p.h0, (size_t)B * 4 * d, dtype, s);
        h0f = p.h0;
    }
    SlstmBwdArgs a{};
    a.wx = wx;
    a.states = states;
    a.grad_states = grad;
    a.g_slot = grad_slot;
    a.r = p.r;
    a.halo = h0f;
    a.halo_stride = 4 * d;
    a.g_wx = g_wx;
    a.gp_partial = p.partial;
    a.gb_partial = g_bias ? p.partial + (size_t)B * p.chain.max_tt * 4 * d : nullptr;
    a.g_h0 = g_h0;
    a.B = B;
    a.T = T;
    a.d = d;
    a.eps = eps;
    a.chain = next_chain(p.chain, T, slstm_tile_steps(), &st->status);
    int rows = B * a.chain.n_tt;
    const int path = kernel_path(dtype, B, T, d);
    cudaError_t e = cudaErrorNotSupported;
    if (path == 2) e = launch_slstm_bwd_pipe(dtype, a, s);
    if (e == cudaSuccess) rows = B;  // the pipelined kernel writes one partial per batch row
    if (e == cudaErrorNotSupported) e = launch_slstm_bwd(dtype, a, false, s);
    if (e != cudaSuccess) return PRB_ERR_LAUNCH;
    if (launch_reduce_partials(p.partial, rows, 4 * d, g_params, s) != cudaSuccess)
        return PRB_ERR_LAUNCH;
    if (g_bias && launch_reduce_partials(a.gb_partial, rows, 4 * d, g_bias, s) != cudaSuccess)
        return PRB_ERR_LAUNCH;
    return PRB_OK;
}

int prb_bwd_slstm(const void* states, const void* wx, const void* r, const void* h0,
                  const void* grad_states, void* g_wx, float* g_params, float* g_h0, int B, int T,
                  int d, int dtype, float eps, void* workspace, size_t workspace_bytes,
                  prb_stats* stats, prb_stream_t stream) {
    return prb_bwd_slstm_ex(states, wx, r, h0, grad_states, -1, g_wx, g_params, nullptr, g_h0, B, T, d, dtype,
                            eps, workspace, workspace_bytes, stats, stream);
}

/* ---- ParaGRU mix='head' -------------------------------------------------------------- */

namespace {
struct HeadPlan {
    float* A;
    float* h0;
    float* buf[2];
    float* gA_part;
    size_t total;
};
HeadPlan plan_head(void* ws, int B, int T, int d, int H, int K) {
    Bump b(ws);
    HeadPlan p;
    const int dh = d / H;
    p.A = b.take<float>((size_t)3 * H * dh * dh);
    p.h0 = b.take<float>((size_t)B * d);
    const size_t n = (size_t)B * T * d;
    p.buf[0] = K > 3 ? b.take<float>(n) : nullptr;
    p.buf[1] = K > 6 ? b.take<float>(n) : nullptr;
    p.gA_part = b.take<float>((size_t)B * 3 * H * dh * dh);
    p.total = b.off + 256;
    return p;
}
bool head_dim_ok(int d, int H) {
    if (H < 1 || d % H) return false;
    const int dh = d / H;
    return dh == 8 || dh == 16 || dh == 32 || dh == 64;
}
}  // namespace

size_t prb_gru_head_workspace_bytes(int B, int T, int d, int n_heads, int max_iters) {
    if (B < 1 || T < 1 || d < 1 || !head_dim_ok(d, n_heads)) return 0;
    return plan_head(nullptr, B, T, d, n_heads, max_iters).total;
}

int prb_newton_gru_head_fused(const void* wx, const void* a_z, const void* a_r, const void* a_n,
                              const void* h0, void* out, int B, int T, int d, int n_heads, int dtype,
                              int max_iters, float omega, int want_residual, void* workspace,
                              size_t workspace_bytes, prb_stats* stats, prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!wx || !a_z || !a_r || !a_n || !out || !stats || B < 1 || T < 1 || d < 1 || max_iters < 0 ||
        max_iters > kMaxIters || bad_dtype(dtype))
        return PRB_ERR_BAD_ARG;
    if (!head_dim_ok(d, n_heads)) return PRB_ERR_UNSUPPORTED;
    const int K = max_iters, H = n_heads, dh = d / H;
    HeadPlan p = plan_head(nullptr, B, T, d, H, K);
    if (int e = check_ws(workspace, workspace_bytes, p.total)) return e;
    p = plan_head(workspace, B, T, d, H, K);
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    cudaMemsetAsync(st, 0, sizeof(DeviceStats), s);
    const size_t asz = (size_t)H * dh * dh;
    to_f32(a_z, p.A, asz, dtype, s);
    to_f32(a_r, p.A + asz, asz, dtype, s);
    to_f32(a_n, p.A + 2 * asz, asz, dtype, s);
    const float* h0f = nullptr;
    if (h0) {
        to_f32(h0, p.h0, (size_t)B * d, dtype, s);
        h0f = p.h0;
    }
    if (K == 0) {
        // the guess itself: one stage with omega = 0 returns H^0 and its residual
        return launch_gru_head_fwd(dtype, wx, p.A, h0f, nullptr, out, true, 1, false, &st->final_bits,
                                   &st->final_bits, B, T, d, H, 0.f, s) == cudaSuccess
                   ? PRB_OK
                   : PRB_ERR_LAUNCH;
    }
    int done = 0, flip = 0;
    const float* hin = nullptr;
    while (done < K) {
        const int n = K - done < 3 ? K - done : 3;
        const bool last = done + n == K;
        void* dst = last ? out : (void*)p.buf[flip];
        if (launch_gru_head_fwd(dtype, wx, p.A, h0f, hin, dst, last, n, last && want_residual,
                                &st->hist_bits[done], &st->final_bits, B, T, d, H, omega, s) != cudaSuccess)
            return PRB_ERR_LAUNCH;
        hin = p.buf[flip];
        flip ^= 1;
        done += n;
    }
    return PRB_OK;
}

int prb_bwd_gru_head(const void* states, const void* wx, const void* a_z, const void* a_r,
                     const void* a_n, const void* h0, const void* grad_states, void* g_wx, float* g_a,
                     float* g_h0, float* mu_out, int B, int T, int d, int n_heads, int dtype, void* workspace,
                     size_t workspace_bytes, prb_stats* stats, prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!states || !wx || !a_z || !a_r || !a_n || !grad_states || !g_wx || !g_a || !stats || B < 1 ||
        T < 1 || d < 1 || bad_dtype(dtype))
        return PRB_ERR_BAD_ARG;
    if (!head_dim_ok(d, n_heads)) return PRB_ERR_UNSUPPORTED;
    const int H = n_heads, dh = d / H;
    HeadPlan p = plan_head(nullptr, B, T, d, H, 0);
    if (int e = check_ws(workspace, workspace_bytes, p.total)) return e;
    p = plan_head(workspace, B, T, d, H, 0);
    cudaMemsetAsync(stats, 0, sizeof(DeviceStats), s);
    const size_t asz = (size_t)H * dh * dh;
    to_f32(a_z, p.A, asz, dtype, s);
    to_f32(a_r, p.A + asz, asz, dtype, s);
    to_f32(a_n, p.A + 2 * asz, asz, dtype, s);
    const float* h0f = nullptr;
    if (h0) {
        to_f32(h0, p.h0, (size_t)B * d, dtype, s);
        h0f = p.h0;
    }
    if (launch_gru_head_bwd(dtype, wx, states, grad_states, p.A, h0f, g_wx, p.gA_part, g_h0, mu_out, B, T, d, H, s) !=
        cudaSuccess)
        return PRB_ERR_LAUNCH;
    return launch_reduce_partials(p.gA_part, B, 3 * H * dh * dh, g_a, s) == cudaSuccess ? PRB_OK
                                                                                         : PRB_ERR_LAUNCH;
}

/* ---- pass-level entry points (time-sharded driver, profiling) ------------------- */

size_t prb_pass_workspace_bytes(int cell, int B, int T, int d) {
    if (B < 1 || T < 1 || d < 1) return 0;
    Bump b(nullptr);
    const bool sl = cell == kCellSlstmDiag;
    const int tile = sl ? (slstm_tile_steps() < slstm_picard_tile_steps() ? slstm_tile_steps()
                                                                           : slstm_picard_tile_steps())
                        : diag_tile_steps();
    plan_chain(b, B, T, d, tile, sl ? 20 : 2);
    b.take<float>((size_t)B * ((T + tile - 1) / tile) * 4 * d);
    return b.off + 256;
}

namespace {
struct PassWs {
    ChainScratch chain;
    float* partial;
};
int pass_ws(int cell, int B, int T, int d, void* ws, size_t ws_bytes, cudaStream_t s, PassWs& out) {
    if (int e = check_ws(ws, ws_bytes, prb_pass_workspace_bytes(cell, B, T, d))) return e;
    Bump b(ws);
    const bool sl = cell == kCellSlstmDiag;
    const int tile = sl ? (slstm_tile_steps() < slstm_picard_tile_steps() ? slstm_tile_steps()
                                                                           : slstm_picard_tile_steps())
                        : diag_tile_steps();
    out.chain = plan_chain(b, B, T, d, tile, sl ? 20 : 2);
    out.partial = b.take<float>((size_t)B * ((T + tile - 1) / tile) * 4 * d);
    cudaMemsetAsync(out.chain.flags, 0, ((size_t)out.chain.n_chains * out.chain.max_tt + kTickets) * 4, s);
    return PRB_OK;
}
}  // namespace

int prb_diag_guess(int cell, const void* wx, const float* params, const float* h0, float* out, int B,
                   int T, int d, int dtype, prb_stream_t stream) {
    if (!wx || !params || !out || B < 1 || T < 1 || d < 1 || bad_dtype(dtype)) return PRB_ERR_BAD_ARG;
    if (!is_diag_cell(cell)) return PRB_ERR_UNSUPPORTED;
    return launch_diag_guess(cell, dtype, true, wx, params, h0, out, B, T, d, (cudaStream_t)stream) ==
                   cudaSuccess
               ? PRB_OK
               : PRB_ERR_LAUNCH;
}

int prb_diag_newton_pass(int cell, const void* wx, const float* params, const float* hin,
                         const float* halo, const float* carry_in, void* hout, float* tail_out,
                         float* agg_out, int mode, int B, int T, int d, int dtype, float omega,
                         void* workspace, size_t workspace_bytes, prb_stats* stats, int hist_slot,
                         prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!wx || !params || !hin || !stats || B < 1 || T < 1 || d < 1 || bad_dtype(dtype) || mode < 0 ||
        mode > 2 || hist_slot < 0 || hist_slot >= kMaxIters)
        return PRB_ERR_BAD_ARG;
    if (!is_diag_cell(cell)) return PRB_ERR_UNSUPPORTED;
    if ((mode == 2 && !agg_out) || (mode != 2 && !hout)) return PRB_ERR_BAD_ARG;
    PassWs w;
    if (int e = pass_ws(cell, B, T, d, workspace, workspace_bytes, s, w)) return e;
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    DiagFwdArgs a{};
    a.wx = wx;
    a.par = params;
    a.halo = halo;
    a.carry_in = carry_in;
    a.hin = hin;
    a.hout = hout;
    a.tail_out = tail_out;
    a.agg_out = agg_out;
    a.resid_bits = &st->hist_bits[hist_slot];
    a.final_bits = mode == 1 ? &st->final_bits : nullptr;
    a.B = B;
    a.T = T;
    a.d = d;
    a.omega = omega;
    a.chain = next_chain(w.chain, T, diag_tile_steps(), &st->status);
    cudaError_t e = mode == 2 ? launch_diag_newton_agg(cell, dtype, a, s)
                    : diag_pipe(dtype, B, T, d) ? launch_diag_newton_pipe(cell, dtype, a, false, mode == 1, s)
                                                : launch_diag_newton(cell, dtype, a, false, mode == 1, s);
    return e == cudaSuccess ? PRB_OK : PRB_ERR_LAUNCH;
}

int prb_diag_bwd_pass(int cell, const void* states, const void* wx, const float* params,
                      const float* halo, const float* carry_in, const void* grad_states, void* g_wx,
                      float* g_params, float* head_out, float* agg_out, int mode, int B, int T, int d,
                      int dtype, void* workspace, size_t workspace_bytes, prb_stats* stats,
                      prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!states || !wx || !params || !grad_states || !stats || B < 1 || T < 1 || d < 1 ||
        bad_dtype(dtype) || (mode != 0 && mode != 2))
        return PRB_ERR_BAD_ARG;
    if (!is_diag_cell(cell)) return PRB_ERR_UNSUPPORTED;
    if ((mode == 2 && !agg_out) || (mode == 0 && (!g_wx || !g_params))) return PRB_ERR_BAD_ARG;
    PassWs w;
    if (int e = pass_ws(cell, B, T, d, workspace, workspace_bytes, s, w)) return e;
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    const int np = diag_cell_params(cell);
    DiagBwdArgs a{};
    a.wx = wx;
    a.states = states;
    a.grad_states = grad_states;
    a.par = params;
    a.halo = halo;
    a.carry_in = carry_in;
    a.g_wx = g_wx;
    a.gp_partial = w.partial;
    a.g_h0 = head_out;
    a.agg_out = agg_out;
    a.B = B;
    a.T = T;
    a.d = d;
    a.chain = next_chain(w.chain, T, diag_tile_steps(), &st->status);
    const bool pipe = mode == 0 && diag_pipe(dtype, B, T, d);
    if ((pipe ? launch_diag_bwd_pipe(cell, dtype, a, s) : launch_diag_bwd(cell, dtype, a, mode == 2, s)) !=
        cudaSuccess)
        return PRB_ERR_LAUNCH;
    if (mode == 0 &&
        launch_reduce_partials(w.partial, pipe ? B : B * a.chain.n_tt, np * d, g_params, s) != cudaSuccess)
        return PRB_ERR_LAUNCH;
    return PRB_OK;
}

int prb_slstm_picard_pass(const void* wx, const float* r, const float* h_prev, const float* h_halo,
                          const float* carry_in, float* h_out, float* state_out, float* tail_out,
                          float* agg_out, int mode, int n_seg, int seg_len, int B, int T, int d, int dtype,
                          float eps, void* workspace, size_t workspace_bytes, prb_stats* stats,
                          prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!wx || !r || !stats || B < 1 || T < 1 || d < 1 || bad_dtype(dtype) || (mode != 0 && mode != 2) ||
        bad_segments(T, n_seg, seg_len))
        return PRB_ERR_BAD_ARG;
    if ((mode == 2 && !agg_out) || (mode == 0 && !h_out && !state_out)) return PRB_ERR_BAD_ARG;
    PassWs w;
    if (int e = pass_ws(kCellSlstmDiag, B, T, d, workspace, workspace_bytes, s, w)) return e;
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    SlstmPicardArgs a{};
    a.wx = wx;
    a.r = r;
    a.h_prev = h_prev;
    a.h_halo = h_halo;
    a.halo_stride = d;
    a.carry_in = carry_in;
    a.carry_stride = 3 * d;
    a.h_out = h_out;
    a.state_out = state_out;
    a.tail_out = tail_out;
    a.agg_out = agg_out;
    a.B = B;
    a.T = T;
    a.d = d;
    a.eps = eps;
    a.n_seg = n_seg;
    a.seg_len = seg_len;
    a.chain = next_chain(w.chain, T, slstm_picard_tile_steps(), &st->status);
    const int path = kernel_path(dtype, B, T, d);
    cudaError_t e = cudaErrorNotSupported;
    if (mode == 2 && (agg_seg(B, d) || n_seg > 1)) e = launch_slstm_picard_agg_seg(dtype, a, s);
    if (mode == 0 && path == 2) e = launch_slstm_picard_pipe(dtype, a, s);
    if (e == cudaErrorNotSupported && n_seg > 1) return PRB_ERR_UNSUPPORTED;  // look-back kernels: one segment
    if (e == cudaErrorNotSupported) e = launch_slstm_picard(dtype, a, mode == 2, s);
    return e == cudaSuccess ? PRB_OK : PRB_ERR_LAUNCH;
}

int prb_slstm_picard_sweep(const void* wx, const float* r, const float* h_halo, const float* carry_in,
                           float* state_out, float* tail_out, int n_passes, int B, int T, int d,
                           int dtype, float eps, void* workspace, size_t workspace_bytes,
                           prb_stats* stats, prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!wx || !r || !state_out || !stats || B < 1 || T < 1 || d < 1 || n_passes < 1 || bad_dtype(dtype))
        return PRB_ERR_BAD_ARG;
    if (n_passes > slstm_picard_fused_max_passes() || !tma_addressable(dtype, B, T, d))
        return PRB_ERR_UNSUPPORTED;
    PassWs w;
    if (int e = pass_ws(kCellSlstmDiag, B, T, d, workspace, workspace_bytes, s, w)) return e;
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    SlstmPicardArgs a{};
    a.wx = wx;
    a.r = r;
    a.h_halo = h_halo;
    a.halo_stride = d;
    a.carry_in = carry_in;
    a.carry_stride = 3 * d;
    a.state_out = state_out;
    a.tail_out = tail_out;
    a.B = B;
    a.T = T;
    a.d = d;
    a.eps = eps;
    a.chain = next_chain(w.chain, T, slstm_picard_tile_steps(), &st->status);
    const cudaError_t e = launch_slstm_picard_fused(dtype, a, n_passes, s);
    if (e == cudaErrorNotSupported) return PRB_ERR_UNSUPPORTED;
    return e == cudaSuccess ? PRB_OK : PRB_ERR_LAUNCH;
}

int prb_slstm_newton_sweep(const void* wx, const float* r, const float* sin, const float* halo, void* sout,
                           int n_iters, int want_residual, int B, int T, int d, int dtype, float omega,
                           float eps, void* workspace, size_t workspace_bytes, prb_stats* stats,
                           prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!wx || !r || !sin || !sout || !stats || B < 1 || T < 1 || d < 1 || n_iters < 1 || bad_dtype(dtype))
        return PRB_ERR_BAD_ARG;
    if (n_iters > slstm_newton_fused_max_iters() || !tma_addressable(dtype, B, T, d))
        return PRB_ERR_UNSUPPORTED;
    PassWs w;
    if (int e = pass_ws(kCellSlstmDiag, B, T, d, workspace, workspace_bytes, s, w)) return e;
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    SlstmNewtonArgs a{};
    a.wx = wx;
    a.r = r;
    a.sin = sin;
    a.halo = halo;
    a.halo_stride = 4 * d;
    a.sout = sout;
    a.resid_bits = &st->hist_bits[0];
    a.final_bits = want_residual ? &st->final_bits : nullptr;
    a.B = B;
    a.T = T;
    a.d = d;
    a.omega = omega;
    a.eps = eps;
    a.chain = next_chain(w.chain, T, slstm_tile_steps(), &st->status);
    const cudaError_t e = launch_slstm_newton_fused(dtype, a, n_iters, s);
    if (e == cudaErrorNotSupported) return PRB_ERR_UNSUPPORTED;
    return e == cudaSuccess ? PRB_OK : PRB_ERR_LAUNCH;
}

int prb_slstm_newton_pass(const void* wx, const float* r, const float* sin, const float* halo,
                          const float* carry_in, void* sout, float* tail_out, float* agg_out, int mode,
                          int n_seg, int seg_len, int B, int T, int d, int dtype, float omega, float eps,
                          void* workspace, size_t workspace_bytes, prb_stats* stats, int hist_slot,
                          prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!wx || !r || !sin || !stats || B < 1 || T < 1 || d < 1 || bad_dtype(dtype) || mode < 0 ||
        mode > 2 || hist_slot < 0 || hist_slot >= kMaxIters || bad_segments(T, n_seg, seg_len))
        return PRB_ERR_BAD_ARG;
    if ((mode == 2 && !agg_out) || (mode != 2 && !sout)) return PRB_ERR_BAD_ARG;
    PassWs w;
    if (int e = pass_ws(kCellSlstmDiag, B, T, d, workspace, workspace_bytes, s, w)) return e;
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    SlstmNewtonArgs a{};
    a.wx = wx;
    a.r = r;
    a.sin = sin;
    a.halo = halo;
    a.halo_stride = 4 * d;
    a.carry_in = carry_in;
    a.sout = sout;
    a.tail_out = tail_out;
    a.agg_out = agg_out;
    a.resid_bits = &st->hist_bits[hist_slot];
    a.final_bits = mode == 1 ? &st->final_bits : nullptr;
    a.B = B;
    a.T = T;
    a.d = d;
    a.omega = omega;
    a.eps = eps;
    a.n_seg = n_seg;
    a.seg_len = seg_len;
    a.chain = next_chain(w.chain, T, slstm_tile_steps(), &st->status);
    const int path = kernel_path(dtype, B, T, d);
    cudaError_t e = cudaErrorNotSupported;
    if (mode == 2 && (agg_seg(B, d) || n_seg > 1)) e = launch_slstm_newton_agg_seg(dtype, a, s);
    if (mode != 2 && path == 2) e = launch_slstm_newton_pipe(dtype, a, mode == 1, s);
    if (e == cudaErrorNotSupported && n_seg > 1) return PRB_ERR_UNSUPPORTED;
    if (e == cudaErrorNotSupported) e = launch_slstm_newton(dtype, a, mode == 1, mode == 2, s);
    return e == cudaSuccess ? PRB_OK : PRB_ERR_LAUNCH;
}

int prb_slstm_bwd_pass(const void* states, const void* wx, const float* r, const float* halo,
                       const float* carry_in, const void* grad_states, void* g_wx, float* g_params,
                       float* head_out, float* agg_out, int mode, int n_seg, int seg_len, int B, int T,
                       int d, int dtype, float eps, void* workspace, size_t workspace_bytes,
                       prb_stats* stats, prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!states || !wx || !r || !grad_states || !stats || B < 1 || T < 1 || d < 1 || bad_dtype(dtype) ||
        (mode != 0 && mode != 2) || bad_segments(T, n_seg, seg_len))
        return PRB_ERR_BAD_ARG;
    if ((mode == 2 && !agg_out) || (mode == 0 && (!g_wx || !g_params))) return PRB_ERR_BAD_ARG;
    PassWs w;
    if (int e = pass_ws(kCellSlstmDiag, B, T, d, workspace, workspace_bytes, s, w)) return e;
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    SlstmBwdArgs a{};
    a.wx = wx;
    a.states = states;
    a.grad_states = grad_states;
    a.r = r;
    a.halo = halo;
    a.halo_stride = 4 * d;
    a.carry_in = carry_in;
    a.g_wx = g_wx;
    a.gp_partial = w.partial;
    a.g_h0 = head_out;
    a.agg_out = agg_out;
    a.B = B;
    a.T = T;
    a.d = d;
    a.eps = eps;
    a.n_seg = n_seg;
    a.seg_len = seg_len;
    a.chain = next_chain(w.chain, T, slstm_tile_steps(), &st->status);
    int rows = B * a.chain.n_tt;
    const int path = kernel_path(dtype, B, T, d);
    cudaError_t e = cudaErrorNotSupported;
    if (mode == 2 && (agg_seg(B, d) || n_seg > 1)) e = launch_slstm_bwd_agg_seg(dtype, a, s);
    if (mode == 0 && path == 2) e = launch_slstm_bwd_pipe(dtype, a, s);
    if (e == cudaSuccess) rows = B * n_seg;  // one partial row per (segment, batch row)
    if (e == cudaErrorNotSupported && n_seg > 1) return PRB_ERR_UNSUPPORTED;
    if (e == cudaErrorNotSupported) e = launch_slstm_bwd(dtype, a, mode == 2, s);
    if (e != cudaSuccess) return PRB_ERR_LAUNCH;
    if (mode == 0 && launch_reduce_partials(w.partial, rows, 4 * d, g_params, s) != cudaSuccess)
        return PRB_ERR_LAUNCH;
    return PRB_OK;
}

int prb_residual_pass(int cell, const void* wx, const float* params, const float* halo,
                      const void* states, int states_f32, int B, int T, int d, int dtype, float eps,
                      prb_stats* stats, prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!wx || !params || !states || !stats || B < 1 || T < 1 || d < 1 || bad_dtype(dtype))
        return PRB_ERR_BAD_ARG;
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    cudaError_t e;
    if (cell == kCellSlstmDiag)
        e = launch_slstm_residual(dtype, states_f32 != 0, wx, params, halo, 4 * d, states, B, T, d, eps,
                                  &st->final_bits, s);
    else if (is_diag_cell(cell))
        e = launch_diag_residual(cell, dtype, states_f32 != 0, wx, params, halo, states, B, T, d,
                                 &st->final_bits, s);
    else
        return PRB_ERR_UNSUPPORTED;
    return e == cudaSuccess ? PRB_OK : PRB_ERR_LAUNCH;
}

int prb_fold_carries(int monoid, const float* gathered, int rank, int world, int reverse,
                     float* carry_out, int B, int d, prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!gathered || !carry_out || B < 1 || d < 1 || world < 2 || rank < 0 || rank >= world)
        return PRB_ERR_BAD_ARG;
    if ((!reverse && rank == 0) || (reverse && rank == world - 1)) return PRB_ERR_BAD_ARG;
    const int n = B * d, blk = 128, grid = (n + blk - 1) / blk;
    if (monoid == 0)
        fold_carries_kernel<Affine1><<<grid, blk, 0, s>>>(gathered, rank, world, reverse, carry_out, B, d, 2);
    else if (monoid == 1)
        fold_carries_kernel<Affine4><<<grid, blk, 0, s>>>(gathered, rank, world, reverse, carry_out, B, d, 20);
    else if (monoid == 2)
        fold_carries_kernel<PicardMonoid><<<grid, blk, 0, s>>>(gathered, rank, world, reverse, carry_out, B, d, 4);
    else
        return PRB_ERR_BAD_ARG;
    return cudaGetLastError() == cudaSuccess ? PRB_OK : PRB_ERR_LAUNCH;
}

int prb_plan_segments(int cell, int dtype, int B, int T, int d, int* n_seg, int* seg_len) {
    if (!n_seg || !seg_len || B < 1 || T < 1 || d < 1 || bad_dtype(dtype)) return PRB_ERR_BAD_ARG;
    *n_seg = 1;
    *seg_len = T;
    if (cell != kCellSlstmDiag || kernel_path(dtype, B, T, d) != 2) return PRB_OK;
    // aim at two CTAs per SM in ONE wave, keep segments long enough that the two extra tiny
    // launches per pass (segment fold, segment carries) and the pipeline fill stay negligible
    const int chains = B * ((d + kLanes - 1) / kLanes);
    const int target = 2 * sm_count();
    int n = target / chains;  // rounded down: one CTA more than fits costs a whole second wave
    const int min_len = 1024;
    if (n > T / min_len) n = T / min_len;
    if (n < 2) return PRB_OK;
    int len = (T + n - 1) / n;
    len = (len + 63) / 64 * 64;
    *seg_len = len;
    *n_seg = (T + len - 1) / len;
    return PRB_OK;
}

int prb_fold_segments(int monoid, const float* agg, int n_seg, int reverse, float* slot, int B, int d,
                      prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!agg || !slot || n_seg < 1 || B < 1 || d < 1) return PRB_ERR_BAD_ARG;
    const int n = B * d, blk = 128, grid = (n + blk - 1) / blk;
    if (monoid == 0)
        fold_segments_kernel<Affine1><<<grid, blk, 0, s>>>(agg, n_seg, reverse, slot, B, d);
    else if (monoid == 1)
        fold_segments_kernel<Affine4><<<grid, blk, 0, s>>>(agg, n_seg, reverse, slot, B, d);
    else if (monoid == 2)
        fold_segments_kernel<PicardMonoid><<<grid, blk, 0, s>>>(agg, n_seg, reverse, slot, B, d);
    else
        return PRB_ERR_BAD_ARG;
    return cudaGetLastError() == cudaSuccess ? PRB_OK : PRB_ERR_LAUNCH;
}

int prb_segment_carries(int monoid, const float* agg, int n_seg, int reverse, const float* carry0,
                        float* carries, int B, int d, prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!agg || !carries || n_seg < 1 || B < 1 || d < 1) return PRB_ERR_BAD_ARG;
    const int n = B * d, blk = 128, grid = (n + blk - 1) / blk;
    if (monoid == 0)
        segment_carries_kernel<Affine1><<<grid, blk, 0, s>>>(agg, n_seg, reverse, carry0, carries, B, d);
    else if (monoid == 1)
        segment_carries_kernel<Affine4><<<grid, blk, 0, s>>>(agg, n_seg, reverse, carry0, carries, B, d);
    else if (monoid == 2)
        segment_carries_kernel<PicardMonoid><<<grid, blk, 0, s>>>(agg, n_seg, reverse, carry0, carries, B, d);
    else
        return PRB_ERR_BAD_ARG;
    return cudaGetLastError() == cudaSuccess ? PRB_OK : PRB_ERR_LAUNCH;
}

int prb_shard_carries(int monoid, const float* gathered, int slot_rows, int rank, int world, int reverse,
                      const float* agg, int n_seg, float* carry_out, float* carries, float eps, float* h_end,
                      int B, int d, prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!gathered || !carry_out || B < 1 || d < 1 || world < 2 || rank < 0 || rank >= world || n_seg < 1)
        return PRB_ERR_BAD_ARG;
    if ((!reverse && rank == 0) || (reverse && rank == world - 1)) return PRB_ERR_BAD_ARG;
    if (carries && !agg) return PRB_ERR_BAD_ARG;
    const int nv = monoid == 0 ? 2 : (monoid == 1 ? 20 : 4);
    if (slot_rows < nv || (h_end && (monoid != 2 || slot_rows < nv + 1))) return PRB_ERR_BAD_ARG;
    const int n = B * d, blk = 128, grid = (n + blk - 1) / blk;
    if (monoid == 0)
        shard_carries_kernel<Affine1><<<grid, blk, 0, s>>>(gathered, slot_rows, rank, world, reverse, agg, n_seg,
                                                           carry_out, carries, eps, nullptr, B, d);
    else if (monoid == 1)
        shard_carries_kernel<Affine4><<<grid, blk, 0, s>>>(gathered, slot_rows, rank, world, reverse, agg, n_seg,
                                                           carry_out, carries, eps, nullptr, B, d);
    else if (monoid == 2)
        shard_carries_kernel<PicardMonoid><<<grid, blk, 0, s>>>(gathered, slot_rows, rank, world, reverse, agg,
                                                                n_seg, carry_out, carries, eps, h_end, B, d);
    else
        return PRB_ERR_BAD_ARG;
    return cudaGetLastError() == cudaSuccess ? PRB_OK : PRB_ERR_LAUNCH;
}

int prb_residual(int cell, const void* wx, const void* params, const void* h0, const void* states,
                 int B, int T, int d, int dtype, float eps, void* workspace, size_t workspace_bytes,
                 prb_stats* stats, prb_stream_t stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (!wx || !params || !states || !stats || B < 1 || T < 1 || d < 1 || bad_dtype(dtype))
        return PRB_ERR_BAD_ARG;
    if (!is_diag_cell(cell) && cell != kCellSlstmDiag) return PRB_ERR_UNSUPPORTED;
    const int np = cell == kCellSlstmDiag ? 4 : diag_cell_params(cell);
    const int S = cell == kCellSlstmDiag ? 4 : 1;
    Bump b(nullptr);
    b.take<float>((size_t)np * d);
    b.take<float>((size_t)B * S * d);
    const size_t need = b.off + 256;
    if (int e = check_ws(workspace, workspace_bytes, need)) return e;
    Bump bb(workspace);
    float* par = bb.take<float>((size_t)np * d);
    float* h0buf = bb.take<float>((size_t)B * S * d);
    DeviceStats* st = reinterpret_cast<DeviceStats*>(stats);
    cudaMemsetAsync(&st->final_bits, 0, sizeof(unsigned), s);
    to_f32(params, par, (size_t)np * d, dtype, s);
    const float* h0f = nullptr;
    if (h0) {
        to_f32(h0, h0buf, (size_t)B * S * d, dtype, s);
        h0f = h0buf;
    }
    cudaError_t e;
    if (cell == kCellSlstmDiag)
        e = launch_slstm_residual(dtype, false, wx, par, h0f, 4 * d, states, B, T, d, eps, &st->final_bits, s);
    else
        e = launch_diag_residual(cell, dtype, false, wx, par, h0f, states, B, T, d, &st->final_bits, s);
    return e == cudaSuccess ? PRB_OK : PRB_ERR_LAUNCH;
}


int prb_decode_step(int cell, const void* state, const void* wx, const void* params_raw, float cap,
                    const int* block_table, void* out, int B, int d, int dtype, float eps,
                    prb_stream_t stream) {
    if (!state || !wx || !params_raw || !out || B < 1 || d < 1 || bad_dtype(dtype)) return PRB_ERR_BAD_ARG;
    if (!is_diag_cell(cell) && cell != kCellSlstmDiag) return PRB_ERR_UNSUPPORTED;
    return launch_decode_step(cell, dtype, state, wx, params_raw, block_table, out, B, d, cap, eps,
                              (cudaStream_t)stream) == cudaSuccess
               ? PRB_OK
               : PRB_ERR_LAUNCH;
}

/* ---- entry point that allocates nothing ---------------------------------------------- */

// Scratch for prb_bwd_nlru_static.  It is part of the library image: every GPU whose
// context loads this library carries these bytes until the process exits.  In host code the
// name `g_static_scratch` is only a handle for cudaGetSymbolAddress; the address that
// kernels may dereference is the one that call returns for the current device.
static __device__ __align__(256) unsigned char g_static_scratch[PRB_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_static_scratch_addr[kMaxDevices] = {};

// Device address of the static scratch on the current device, resolved once per device.
int static_scratch_address(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return PRB_ERR_LAUNCH;
    if (!g_static_scratch_addr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) return PRB_ERR_LAUNCH;
        g_static_scratch_addr[dev] = p;
    }
    *out = g_static_scratch_addr[dev];
    return PRB_OK;
}
}  // namespace

size_t prb_static_scratch_bytes(void) { return PRB_STATIC_SCRATCH_BYTES; }

int prb_bwd_nlru_static(const void* states, const void* wx, const void* u, const void* h0,
                        const void* grad_states, void* g_wx, float* g_params, float* g_h0, int B,
                        int T, int d, int dtype, prb_stats* stats, prb_stream_t stream) {
    if (B < 1 || T < 1 || d < 1) return PRB_ERR_BAD_ARG;
    // the same layout the workspace-taking entry point uses; refuse what does not fit
    if (plan_diag_bwd(nullptr, kCellNlru, B, T, d).total > PRB_STATIC_SCRATCH_BYTES)
        return PRB_ERR_TOO_LARGE;
    void* scratch = nullptr;
    if (int e = static_scratch_address(&scratch)) return e;
    // run_diag_bwd clears the chain flags, the ticket counters and the statistics block before
    // the kernels start; everything else in the scratch is written before it is read.
    const void* pars[3] = {u, nullptr, nullptr};
    return run_diag_bwd(kCellNlru, states, wx, pars, h0, grad_states, g_wx, g_params, g_h0, B, T, d,
                        dtype, scratch, PRB_STATIC_SCRATCH_BYTES, stats, (cudaStream_t)stream);
}

}  // extern "C"
