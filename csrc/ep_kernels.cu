// Dispatch / combine kernels for sm_100a: stage, plan, pull, push, reduce, barrier.
// See ep_kernels.hpp for the protocol.  All waits are bounded (prim.cuh); nothing traps.
#include "ep_kernels.hpp"
#include "prim.cuh"

namespace nep {
namespace {

constexpr unsigned kFull = 0xffffffffu;
constexpr int kStageThreads = 512;
constexpr int kPlanThreads = 256;
constexpr int kReduceThreads = 512;
constexpr int kZeroBytes = 2048;  // zero source of the padding rows
constexpr int kTagStage = 1, kTagPlan = 2, kTagPull = 3, kTagPush = 4, kTagReduce = 5, kTagBarrier = 6;

__device__ __forceinline__ char* window(const CommonParams& c, int r) { return static_cast<char*>(c.peers[r]); }
__device__ __forceinline__ int* ctrl_words(const CommonParams& c) {
    return reinterpret_cast<int*>(window(c, c.rank) + c.layout.ctrl_offset);
}
__device__ __forceinline__ StatusRef status_of(const CommonParams& c) { return StatusRef{c.status_dev, c.status_host}; }
__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// The block that takes the last ticket runs the tail of a kernel; the counter is reset by it.
__device__ __forceinline__ bool take_last_ticket(int* ticket) {
    __shared__ int last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = (atomicAdd(ticket, 1) == int(gridDim.x) - 1);
    __syncthreads();
    if (last) __threadfence();
    return last != 0;
}

// Single-launch paths: the block that took the last ticket runs the peer barrier and then tells the other
// blocks of its rank the outcome through one word: +tag = go, -tag = failed (tag derives from the epoch, never 0).
__device__ __forceinline__ int go_tag(uint64_t epoch) { return int(epoch & 0x3fffffff) | 0x40000000; }

__device__ __forceinline__ void publish_go(int* ctrl, uint64_t epoch, bool ok, int word = WindowLayout::kGoWord) {
    const int want = go_tag(epoch);
    __threadfence();
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(ctrl + word), "r"(ok ? want : -want) : "memory");
}

// Called by every thread of a block; thread 0 polls (bounded), the block gets the outcome.
__device__ bool wait_go(int* ctrl, uint64_t epoch, uint64_t timeout_ns, StatusRef status, uint32_t tag, int word = WindowLayout::kGoWord) {
    __shared__ int s_go;
    if (threadIdx.x == 0) {
        const int want = go_tag(epoch);
        const uint64_t start = global_timer_ns();
        int seen = 0;
        for (;;) {
            seen = ld_acquire_gpu(ctrl + word);
            if (seen == want || seen == -want) break;
            __nanosleep(32);
            if (global_timer_ns() - start > 2 * timeout_ns) {
                report(status, kBarrierTimeout, 0xffffu, tag);
                seen = -want;
                break;
            }
        }
        s_go = seen == want;
    }
    __syncthreads();
    return s_go != 0;
}

// ------------------------------------------------------------------------------------------
// stage: copy this rank's tokens (x + gate weights) into its own window, snapshot and count the
// routing, send the per-destination counts to the peers, peer barrier, derive N / C / offsets.
// ------------------------------------------------------------------------------------------
// Returns true when the peer barrier succeeded (only meaningful to every block in fused mode).
__device__ bool stage_body(const StageParams& p) {
    extern __shared__ int s_counts[];  // [R + E]
    const WindowLayout& L = p.c.layout;
    const int R = L.ranks, K = L.topk, H = L.hidden, Le = L.local_experts;
    const int E = int(L.num_experts);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wpb = blockDim.x >> 5;
    const int gw = blockIdx.x * wpb + warp, GW = gridDim.x * wpb;
    char* win = window(p.c, p.c.rank);
    int* ctrl = ctrl_words(p.c);
    int* count_acc = ctrl + L.ctrl_count_acc();
    const StatusRef status = status_of(p.c);

    if (p.fresh) {
        for (int i = tid; i < R + E; i += blockDim.x) s_counts[i] = 0;
        __syncthreads();
    }
    char* rows = win + L.stage_rows_offset + int64_t(p.parity) * L.stage_rows_stride;
    // this rank's slice of every receiver's routing table
    const int64_t routing_slice = L.routing_in_offset + int64_t(p.parity) * L.routing_in_stride + int64_t(p.c.rank) * L.max_tokens * K * 4;
    const int64_t rb = L.row_bytes();
    const int vecs = H / 8;  // 16-byte chunks per row

    auto stamp = [&](int slot) {
        if (p.trace != nullptr && tid == 0) atomicMax(p.trace + slot, global_timer_ns());
    };
    if (p.trace != nullptr && tid == 0) atomicMin(p.trace, global_timer_ns());

    // ---- fresh dispatch, step 1: snapshot, validate, publish and count the routing (one warp per token).  The
    // counts are what every rank and the host wait for, so they go first; the rows follow underneath the exchange.
    bool runs_tail = false;
    if (p.fresh) {
        for (int t = gw; t < p.tokens; t += GW) {
            int e = -1;
            bool valid = false;
            if (lane < K) {
                const int64_t raw = p.topk[int64_t(t) * K + lane];
                p.snapshot[int64_t(t) * K + lane] = raw;
                if (raw >= 0 && raw < E) {
                    e = int(raw);
                    valid = true;
                } else if (raw != -1) {
                    report(status, kBadExpertId, uint32_t(t), kTagStage);
                }
                // Publish the routing to every rank (itself included): receivers plan from local memory.
                for (int d = 0; d < R; ++d) reinterpret_cast<int*>(window(p.c, d) + routing_slice)[int64_t(t) * K + lane] = e;
            }
            const unsigned vmask = __ballot_sync(kFull, valid);
            const int d = valid ? e / Le : -1;
            if (valid) {
                atomicAdd(&s_counts[R + e], 1);
                const unsigned same = __match_any_sync(vmask, d);
                if (lane == __ffs(same) - 1) atomicAdd(&s_counts[d], 1);
            }
            const unsigned dmask = __reduce_or_sync(kFull, valid ? (1u << d) : 0u);
            if (lane < R) {
                const bool goes = (dmask >> lane) & 1u;
                p.dst_slots[int64_t(t) * R + lane] = goes ? int64_t(t) : int64_t(-1);
                // rows this rank sends to destination `lane` out of the token's chunk of 32: the receivers turn these
                // into row offsets, so that receive rows are ordered by (source rank, source token)
                if (goes) atomicAdd(ctrl + L.ctrl_chunk_acc() + int64_t(lane) * L.chunks_per_rank() + (t >> 5), 1);
            }
        }
        __syncthreads();
        for (int i = tid; i < R + E; i += blockDim.x)
            if (s_counts[i] != 0) atomicAdd(&count_acc[i], s_counts[i]);
        runs_tail = take_last_ticket(ctrl + WindowLayout::kTicketStage);
        stamp(1);
    }

    __shared__ int s_ok;
    __shared__ int s_total[2];

    auto copy_rows = [&]() {
        // ---- rows: x and gate weights into this rank's staging area.  Work item = one quarter of a token row, so that
        // even a few thousand tokens spread over the whole grid and every lane keeps up to eight 16-byte loads in flight.
        if (!p.skip_copy) {
            constexpr int kParts = 4;
            const int per_part = (vecs + kParts - 1) / kParts;
            for (int item = gw; item < p.tokens * kParts; item += GW) {
                const int t = item / kParts, q = item % kParts;
                const int4* src = reinterpret_cast<const int4*>(p.x + int64_t(t) * H);
                int4* dst = reinterpret_cast<int4*>(rows + int64_t(t) * rb);
                const int end = min(vecs, (q + 1) * per_part);
                for (int i = q * per_part + lane; i < end; i += 256) {
                    int4 v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (i + j * 32 < end) v[j] = ld_nc_v4(src + i + j * 32);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (i + j * 32 < end) dst[i + j * 32] = v[j];
                }
                if (q == 0 && lane < K) {
                    const float w = p.weights != nullptr ? p.weights[int64_t(t) * K + lane] : 0.f;
                    reinterpret_cast<float*>(rows + int64_t(t) * rb + wire_weights_offset(H))[lane] = w;
                }
            }
        }
    };

    // The tail: run by ONE block per rank (the one that took the last ticket of the counting step, or of the copy in a
    // cached dispatch).  Returns whether the peer barrier succeeded.
    auto tail = [&]() -> bool {
        // ---- tail: one block per rank
        const int msg = int(L.msg_ints());
        if (p.fresh) {
            for (int i = tid; i < R * msg; i += blockDim.x) {
                const int d = i / msg, j = i % msg;
                const int v = j == 0 ? __ldcg(count_acc + d) : j == 1 ? p.tokens : __ldcg(count_acc + R + d * Le + (j - 2));
                int* remote =
                    reinterpret_cast<int*>(window(p.c, d) + L.counts_in_offset + int64_t(p.parity) * L.counts_in_stride) + p.c.rank * msg + j;
                st_relaxed_sys(remote, v);
            }
            for (int d = tid; d < R; d += blockDim.x) p.send_counts[d] = __ldcg(count_acc + d);
            // per-chunk row counts go to their destination (the accumulators are cleared for the next dispatch)
            const int cps = int(L.chunks_per_rank()), my_chunks = (p.tokens + 31) / 32;
            int* chunk_acc = ctrl + L.ctrl_chunk_acc();
            for (int i = tid; i < R * my_chunks; i += blockDim.x) {
                const int d = i / my_chunks, c = i % my_chunks;
                int* remote = reinterpret_cast<int*>(window(p.c, d) + L.chunks_in_offset + int64_t(p.parity) * L.chunks_in_stride) + p.c.rank * cps + c;
                st_relaxed_sys(remote, __ldcg(chunk_acc + d * cps + c));
                chunk_acc[d * cps + c] = 0;
            }
            __syncthreads();
            for (int i = tid; i < R + E; i += blockDim.x) count_acc[i] = 0;
        }
        if (tid == 0) ctrl[WindowLayout::kTicketStage] = 0;
        if (R > 1) {
            __threadfence_system();
            __syncthreads();
            if (warp == 0) {
                const bool ok = peer_barrier_warp(p.c.peers, p.c.rank, R, L.signal_offset, p.epoch, p.c.timeout_ns, status, kTagStage);
                if (lane == 0) s_ok = ok;
            }
        } else {
            // a single-rank group has nobody to wait for: its own messages are ordered by the block barrier below
            __threadfence();
            if (tid == 0) s_ok = 1;
        }
        __syncthreads();
        stamp(3);
        if (p.fused && !p.fresh) {
            if (tid == 0) publish_go(ctrl, p.epoch, s_ok != 0);
            return s_ok != 0;
        }
        if (!p.fresh) return s_ok != 0;
        if (!s_ok) {
            if (tid == 0) {
                p.mailbox[1] = -2;
                p.mailbox[0] = -2;
                __threadfence_system();
                if (p.fused) publish_go(ctrl, p.epoch, false);
            }
            return false;
        }
        const int* in = reinterpret_cast<const int*>(win + L.counts_in_offset + int64_t(p.parity) * L.counts_in_stride);
        // Phase 1 (all threads): per local expert, sum the sources' counts and round up to the alignment.
        // The padded sizes reuse the dynamic shared array (R + E ints >= L ints).
        int* s_padded = s_counts;
        for (int l = tid; l < Le; l += blockDim.x) {
            int cnt = 0;
            for (int src = 0; src < R; ++src) cnt += ld_relaxed_sys(in + src * msg + 2 + l);
            p.expert_counts[l] = cnt;
            ctrl[L.ctrl_expert_counts() + l] = cnt;
            ctrl[L.ctrl_expert_cursor() + l] = 0;
            s_padded[l] = (cnt + p.alignment - 1) / p.alignment * p.alignment;
        }
        __syncthreads();
        if (warp == 0) {
            // receive rows by source: inclusive prefix (R <= 32)
            const int n = lane < R ? ld_relaxed_sys(in + lane * msg) : 0;
            const int incl = warp_inclusive_sum(n);
            if (lane < R) {
                p.recv_rank_prefix[lane] = incl;
                ctrl[L.ctrl_recv_prefix() + lane] = incl - n;
                ctrl[L.ctrl_src_tokens() + lane] = ld_relaxed_sys(in + lane * msg + 1);
            }
            if (lane == R - 1) {
                ctrl[L.ctrl_recv_prefix() + R] = incl;
                s_total[0] = incl;
            }
        } else if (warp == 1) {
            // Phase 2: exclusive scan of the padded sizes in waves of 32 (shared memory only)
            int carry = 0;
            for (int base = 0; base < Le; base += 32) {
                const int l = base + lane;
                const int padded = l < Le ? s_padded[l] : 0;
                const int incl = warp_inclusive_sum(padded);
                if (l < Le) {
                    const int off = carry + incl - padded;
                    p.expert_offsets[l] = off;
                    ctrl[L.ctrl_expert_offsets() + l] = off;
                }
                carry += __shfl_sync(kFull, incl, 31);
            }
            if (lane == 0) {
                p.expert_offsets[Le] = carry;
                ctrl[L.ctrl_expert_offsets() + Le] = carry;
                s_total[1] = carry;
            }
        }
        // Every source's per-chunk row counts become exclusive prefixes: chunk c of source s starts at receive row
        // recv_prefix[s] + chunk_prefix[s][c].  The total must equal the source's announced row count.
        {
            const int cps = int(L.chunks_per_rank());
            int* chunks = reinterpret_cast<int*>(win + L.chunks_in_offset + int64_t(p.parity) * L.chunks_in_stride);
            for (int s = warp; s < R; s += wpb) {
                const int n_chunks = (ld_relaxed_sys(in + s * msg + 1) + 31) / 32;
                int carry = 0;
                for (int base = 0; base < n_chunks; base += 32) {
                    const int c = base + lane;
                    const int v = c < n_chunks ? ld_relaxed_sys(chunks + s * cps + c) : 0;
                    const int incl = warp_inclusive_sum(v);
                    if (c < n_chunks) chunks[s * cps + c] = carry + incl - v;
                    carry += __shfl_sync(kFull, incl, 31);
                }
                if (lane == 0 && carry != ld_relaxed_sys(in + s * msg)) report(status, kSlotOverflow, uint32_t(s), kTagStage);
            }
        }
        __syncthreads();
        if (tid == 0) {
            __threadfence_system();
            p.mailbox[1] = s_total[1];
            p.mailbox[0] = s_total[0];
            __threadfence_system();
            if (p.fused) publish_go(ctrl, p.epoch, true);  // the other blocks of a single-launch dispatch go on to plan
        }
        stamp(4);
        return true;
    };

    if (p.fresh) {
        // The count exchange comes first: every rank and the host wait for it.  The rows are staged underneath it by all
        // the other blocks; the tail block copies its own small share afterwards.
        bool ok = true;
        if (runs_tail) ok = tail();
        copy_rows();
        // The block that finishes its rows last tells every peer that this rank's rows are staged; the receivers'
        // pull waits for these signals, nobody waits here.
        if (take_last_ticket(ctrl + WindowLayout::kTicketCopy)) {
            if (tid == 0) ctrl[WindowLayout::kTicketCopy] = 0;
            if (R > 1) {  // a single-rank group stages nothing and its pull waits for no signal
                __threadfence_system();
                __syncthreads();
                if (warp == 0) peer_signal_warp(p.c.peers, p.c.rank, R, L.data_signal_offset, p.epoch);
            }
        }
        stamp(2);
        if (runs_tail) return ok;
        // single-launch fresh dispatch: wait for the tail block's prefixes before planning
        if (!p.fused) return false;
        return wait_go(ctrl, p.epoch, p.c.timeout_ns, status, kTagStage);
    }
    copy_rows();
    if (!take_last_ticket(ctrl + WindowLayout::kTicketStage)) {
        if (!p.fused) return false;
        return wait_go(ctrl, p.epoch, p.c.timeout_ns, status, kTagStage);
    }
    return tail();
}

// ------------------------------------------------------------------------------------------
// plan (fresh dispatch): every receiver scans the routing all sources wrote into its window, 32 tokens at a time,
// keeps the tokens that chose one of its experts, and assigns a receive row (grouped by source
// rank) and, in the expert-major layout, one slot per local choice.
// ------------------------------------------------------------------------------------------
__device__ void plan_body(const PlanParams& p) {
    extern __shared__ int s_chunk[];  // [warps][32*K]
    const WindowLayout& L = p.c.layout;
    const int R = L.ranks, K = L.topk, Le = L.local_experts;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    const int gw = blockIdx.x * wpb + warp, GW = gridDim.x * wpb;
    int* ctrl = ctrl_words(p.c);
    const int* prefix = ctrl + L.ctrl_recv_prefix();
    const int* src_tokens = ctrl + L.ctrl_src_tokens();
    const int* eoff = ctrl + L.ctrl_expert_offsets();
    int* expert_cursor = ctrl + L.ctrl_expert_cursor();
    const int* chunk_prefix = reinterpret_cast<const int*>(window(p.c, p.c.rank) + L.chunks_in_offset + int64_t(p.parity) * L.chunks_in_stride);
    int* meta = reinterpret_cast<int*>(window(p.c, p.c.rank) + L.meta_scratch_offset);
    int* mine = s_chunk + warp * 32 * K;
    const StatusRef status = status_of(p.c);
    const int cps = int((L.max_tokens + 31) / 32);
    const int lo = p.c.rank * Le;
    int* slot_scratch = reinterpret_cast<int*>(window(p.c, p.c.rank) + L.slot_scratch_offset);
    if (p.expand) {
        // alignment gaps of the expert-major layout hold no row
        const int* ecnt = ctrl + L.ctrl_expert_counts();
        for (int l = gw; l < Le; l += GW)
            for (int slot = eoff[l] + ecnt[l] + lane; slot < eoff[l + 1]; slot += 32)
                if (slot < L.slot_scratch_ints) slot_scratch[slot] = -1;
    }

    for (int c = gw; c < R * cps; c += GW) {
        const int s = c / cps, tok0 = (c % cps) * 32;
        const int Ts = src_tokens[s];
        if (tok0 >= Ts) continue;
        const int n_tok = min(32, Ts - tok0);
        const int n = n_tok * K;
        const int* remote = reinterpret_cast<const int*>(window(p.c, p.c.rank) + L.routing_in_offset + int64_t(p.parity) * L.routing_in_stride) +
                            (int64_t(s) * L.max_tokens + tok0) * K;
        __syncwarp();
        for (int base = 0; base < n; base += 256) {
            int v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = base + j * 32 + lane;
                v[j] = i < n ? ld_relaxed_sys(remote + i) : -1;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = base + j * 32 + lane;
                if (i < n) mine[i] = v[j];
            }
        }
        __syncwarp();
        bool has = false;
        if (lane < n_tok)
            for (int k = 0; k < K; ++k) {
                const int e = mine[lane * K + k];
                has |= (e >= lo && e < lo + Le);
            }
        const unsigned hm = __ballot_sync(kFull, has);
        if (hm == 0) continue;
        // rows of a source are ordered by token: the chunk's first row comes from the prefix the stage kernel built
        const int base_row = chunk_prefix[s * cps + (tok0 >> 5)];
        if (has) {
            const int row = prefix[s] + base_row + __popc(hm & lanemask_lt());
            if (row >= prefix[s + 1]) {
                report(status, kSlotOverflow, uint32_t(row), kTagPlan);
            } else {
                int* m = meta + int64_t(row) * (K + 2);
                m[0] = s;
                m[1] = tok0 + lane;
                // Eight choices at a time: all slot atomics of a group are issued before any result
                // is consumed, so their latencies overlap.
                for (int k0 = 0; k0 < K; k0 += 8) {
                    int le[8], got[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int e = k0 + j < K ? mine[lane * K + k0 + j] : -1;
                        le[j] = (e >= lo && e < lo + Le) ? e - lo : -1;
                        got[j] = (p.expand && le[j] >= 0) ? atomicAdd(&expert_cursor[le[j]], 1) : 0;
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (k0 + j >= K) break;
                        int v = -1;
                        if (le[j] >= 0) {
                            v = p.expand ? eoff[le[j]] + got[j] : le[j];
                            if (p.expand && v >= eoff[le[j] + 1]) {
                                report(status, kSlotOverflow, uint32_t(v), kTagPlan);
                                v = -1;
                            }
                            if (p.expand && v >= 0 && v < L.slot_scratch_ints) slot_scratch[v] = row * K + k0 + j;
                        }
                        m[2 + k0 + j] = v;
                    }
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// Ring of row buffers private to one warp, filled by bulk loads that complete on mbarriers.
// ------------------------------------------------------------------------------------------
struct Ring {
    char* buf;
    uint64_t* bars;
    int stages;
    int64_t pitch;
    uint32_t parity;  // bit s = parity of the next phase to wait for on stage s
    __device__ __forceinline__ char* slot(int i) const { return buf + int64_t(i % stages) * pitch; }
    __device__ __forceinline__ uint64_t* bar(int i) const { return bars + (i % stages); }
    // Wait for the load issued into item i's stage.  Only stages that really received a load may be
    // waited on: the parity advances per completed wait, not per item, so skipped items are harmless.
    __device__ __forceinline__ bool wait(int i, uint64_t timeout_ns) {
        const int s = i % stages;
        bool ok = mbar_wait(bars + s, (parity >> s) & 1u, timeout_ns);
        ok = __all_sync(0xffffffffu, ok);
        parity ^= 1u << s;
        return ok;
    }
};

__device__ __forceinline__ Ring make_ring(char* smem, int warps, int stages, int64_t row_bytes) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t pitch = align_up(row_bytes, 128);
    Ring r;
    r.buf = smem + int64_t(warp) * stages * pitch;
    r.bars = reinterpret_cast<uint64_t*>(smem + int64_t(warps) * stages * pitch) + warp * stages;
    r.stages = stages;
    r.pitch = pitch;
    r.parity = 0;
    if (lane == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(r.bars + s, 1);
        mbar_init_fence();
        fence_proxy_async_smem();
    }
    __syncwarp();
    return r;
}


// Receive rows are stored grouped by source rank.  Walking them in storage order would make every
// receiver talk to the same source at the same time (one GPU's NVLink port serving all others).
// Instead item v visits the sources round-robin, starting after the own rank:
//   source s = (rank + 1 + v % R) % R,  j = v / R,  row = first_row(s) + j   (skipped when j >= rows(s)).
struct SourceWalk {
    int first, count;  // lane s: first receive row and row count of source s
    int items;         // R * max_s count
    int rank, ranks;
    __device__ __forceinline__ bool locate(int v, int& row) const {
        const int s = (rank + 1 + v % ranks) % ranks;
        const int j = v / ranks;
        const int f = __shfl_sync(0xffffffffu, first, s);
        const int c = __shfl_sync(0xffffffffu, count, s);
        row = f + j;
        return j < c;
    }
};
__device__ __forceinline__ SourceWalk make_walk(const int64_t* inclusive_prefix, int rank, int ranks) {
    const int lane = threadIdx.x & 31;
    SourceWalk w;
    const int incl = lane < ranks ? int(inclusive_prefix[lane]) : 0;
    const int prev = lane > 0 && lane < ranks ? int(inclusive_prefix[lane - 1]) : 0;
    w.first = prev;
    w.count = lane < ranks ? incl - prev : 0;
    int mx = w.count;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    w.items = mx * ranks;
    w.rank = rank;
    w.ranks = ranks;
    return w;
}

// ------------------------------------------------------------------------------------------
// pull: for every receive row, bulk-load the staged row from its source rank (NVLink or local)
// into shared memory and bulk-store it to its final place(s): row r (compact) or every
// expert-major slot of the row (expanded).  Gaps of the expert-major layout are zero-filled here.
// ------------------------------------------------------------------------------------------
__device__ void pull_body(const PullParams& p) {
    extern __shared__ __align__(128) char s_ring[];
    const WindowLayout& L = p.c.layout;
    const int R = L.ranks, K = L.topk, H = L.hidden, Le = L.local_experts;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    const int gw = blockIdx.x * wpb + warp, GW = gridDim.x * wpb;
    const int64_t rb = L.row_bytes();
    const StatusRef status = status_of(p.c);
    const int MW = K + 2;
    Ring ring = make_ring(s_ring, wpb, p.stages, rb);
    const int S = p.stages;
    if (p.data_epoch != 0) {
        // A fresh dispatch stages its rows underneath the count exchange: every source signals when its rows are in place.
        __shared__ int s_staged;
        if (warp == 0) {
            const bool ok = peer_wait_warp(p.c.peers, p.c.rank, R, L.data_signal_offset, p.data_epoch, p.c.timeout_ns, status, kTagPull);
            if (lane == 0) s_staged = ok;
        }
        __syncthreads();
        if (!s_staged) return;
        fence_proxy_async();
    }
    const SourceWalk walk = make_walk(p.recv_rank_prefix, p.c.rank, R);
    const bool slot_order = p.slot_src != nullptr;
    const int n_items = slot_order ? p.capacity : walk.items;
    const int n_my = n_items > gw ? (n_items - gw + GW - 1) / GW : 0;
    // item -> receive row to transfer now (false: nothing to do for this item)
    auto locate = [&](int item, int& r) {
        if (!slot_order) return walk.locate(item, r);
        const int a = p.slot_src[item];
        r = a >= 0 ? a / K : 0;
        const int v = (a >= 0 && lane < K) ? p.meta[int64_t(r) * MW + 2 + lane] : -1;
        int lowest = v >= 0 ? v : 0x7fffffff;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) lowest = min(lowest, __shfl_xor_sync(kFull, lowest, d));
        return a >= 0 && lowest == item;
    };

    auto issue = [&](int i) {
        int r;
        const bool live = locate(gw + i * GW, r);
        if (lane == 0 && live) {
            int src = p.meta[int64_t(r) * MW], tok = p.meta[int64_t(r) * MW + 1];
            if (src < 0 || src >= R || tok < 0 || tok >= L.max_tokens) {
                report(status, kBadMetadata, uint32_t(r), kTagPull);
                src = p.c.rank;
                tok = 0;
            }
            if (src == p.c.rank && p.x_local != nullptr) {
                mbar_expect_tx(ring.bar(i), uint32_t(H) * 2u);
                bulk_load(ring.slot(i), p.x_local + int64_t(tok) * H, uint32_t(H) * 2u, ring.bar(i));
            } else {
                const char* from = window(p.c, src) + L.stage_rows_offset + int64_t(p.parity) * L.stage_rows_stride + int64_t(tok) * rb;
                mbar_expect_tx(ring.bar(i), uint32_t(rb));
                bulk_load(ring.slot(i), from, uint32_t(rb), ring.bar(i));
            }
        }
    };
    for (int i = 0; i < min(S - 1, n_my); ++i) issue(i);

    // Gaps between an expert's last real row and the next expert's first slot: zero rows are bulk
    // stores from a small zero buffer behind the rings (few instructions, no LSU store traffic).
    char* zero_buf = s_ring + (align_up(rb, 128) + 8) * int64_t(wpb) * S;
    zero_buf = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(zero_buf) + 127) & ~uintptr_t(127));
    if (p.expand && p.zero_padding) {
        for (int i = threadIdx.x; i < kZeroBytes / 16; i += blockDim.x) reinterpret_cast<int4*>(zero_buf)[i] = make_int4(0, 0, 0, 0);
        fence_proxy_async_smem();
        __syncthreads();
    }
    if (p.expand) {
        // Gap geometry is read 32 experts at a time (one coalesced load per lane) and handed round by
        // shuffles: a scalar walk over the experts would cost one global-load latency per expert and warp.
        int base = 0;
        for (int l0 = 0; l0 < Le; l0 += 32) {
          const int my_l = l0 + lane;
          const int my_gs = my_l < Le ? int(p.expert_offsets[my_l] + p.expert_counts[my_l]) : 0;
          const int my_len = my_l < Le ? int(p.expert_offsets[my_l + 1]) - my_gs : 0;
          const int in_wave = min(32, Le - l0);
          for (int li = 0; li < in_wave; ++li) {
            const int gs = __shfl_sync(kFull, my_gs, li);
            const int len = __shfl_sync(kFull, my_len, li);
            int first = (gw - base) % GW;
            if (first < 0) first += GW;
            for (int j = first; j < len; j += GW) {
                const int64_t row = gs + j;
                if (p.zero_padding) {
                    if (lane == 0) {
                        char* dst = reinterpret_cast<char*>(p.x_out + row * H);
                        for (int at = 0; at < H * 2; at += kZeroBytes) bulk_store(dst + at, zero_buf, uint32_t(min(kZeroBytes, H * 2 - at)));
                        bulk_commit();
                        if (p.w_out != nullptr) p.w_out[row] = 0.f;
                    }
                    if (p.tile_ready != nullptr) bulk_wait<0>();
                }
                if (lane == 0 && p.slot_map != nullptr) p.slot_map[row] = -1;
                if (p.tile_ready != nullptr) {
                    fence_proxy_async();
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) red_release_gpu_add(p.tile_ready + int(row / 128), 1);
                }
            }
            base = (base + len) % GW;
          }
        }
    }

    // With tile counters, a row is announced one iteration late: after the bulk group that stored it
    // has fully completed (not only been read from shared memory).
    const bool announce = p.tile_ready != nullptr && p.expand;
    int announced_slot = -1;
    auto retire_previous = [&]() {
        if (announce) {
            bulk_wait<1>();
            if (announced_slot >= 0) {
                fence_proxy_async();
                red_release_gpu_add(p.tile_ready + announced_slot / 128, 1);
            }
        } else {
            bulk_wait_read<1>();
        }
    };
    for (int i = 0; i < n_my; ++i) {
        int r;
        if (!locate(gw + i * GW, r)) {
            bulk_commit();
            retire_previous();
            announced_slot = -1;
            __syncwarp();
            if (i + S - 1 < n_my) issue(i + S - 1);
            continue;
        }
        if (!ring.wait(i, p.c.timeout_ns)) {
            if (lane == 0) report(status, kCopyTimeout, uint32_t(gw), kTagPull);
            break;
        }
        const int* m = p.meta + int64_t(r) * MW;
        const int v = lane < K ? m[2 + lane] : -1;
        const char* st = ring.slot(i);
        const float* st_w = reinterpret_cast<const float*>(st + wire_weights_offset(H));
        if (m[0] == p.c.rank && p.x_local != nullptr && p.w_local != nullptr) st_w = p.w_local + int64_t(m[1]) * K;
        if (p.expand) {
            if (v >= 0) {
                bulk_store(p.x_out + int64_t(v) * H, st, uint32_t(H) * 2u);
                if (p.w_out != nullptr) p.w_out[v] = st_w[lane];
                if (p.slot_map != nullptr) p.slot_map[v] = r * K + lane;
            }
        } else {
            if (lane == 0) bulk_store(p.x_out + int64_t(r) * H, st, uint32_t(H) * 2u);
            if (lane < K) {
                p.topk_out[int64_t(r) * K + lane] = v;
                if (p.w_out != nullptr) p.w_out[int64_t(r) * K + lane] = st_w[lane];
            }
        }
        if (p.write_meta) {
            for (int j = lane; j < MW; j += 32) p.meta_out[int64_t(r) * MW + j] = m[j];
        }
        bulk_commit();
        retire_previous();
        announced_slot = p.expand ? v : -1;
        __syncwarp();
        if (i + S - 1 < n_my) issue(i + S - 1);
    }
    bulk_wait<0>();
    if (announce && announced_slot >= 0) {
        fence_proxy_async();
        red_release_gpu_add(p.tile_ready + announced_slot / 128, 1);
    }
}

// ------------------------------------------------------------------------------------------
// combine: one launch.  Transfer warps return expert outputs to the source ranks' partitions and flag every
// row on arrival; reduce warps sum a source token once all of its rows are flagged.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ char* ret_row(const CommonParams& c, int src, int part, int tok) {
    const WindowLayout& L = c.layout;
    return window(c, src) + L.ret_offset + (int64_t(part) * L.max_tokens + tok) * L.hidden * 2;
}
__device__ __forceinline__ float* ret_w_row(const CommonParams& c, int src, int tok) {
    const WindowLayout& L = c.layout;
    return reinterpret_cast<float*>(window(c, src) + L.ret_w_offset) + int64_t(tok) * L.topk;
}
__device__ __forceinline__ uint32_t* ret_flag(const CommonParams& c, int src, int part, int tok) {
    const WindowLayout& L = c.layout;
    return reinterpret_cast<uint32_t*>(window(c, src) + L.ret_flag_offset) + int64_t(part) * L.max_tokens + tok;
}
// Value a combine writes into the arrival flags: never 0 (a fresh window), different for consecutive combines.
__device__ __forceinline__ uint32_t combine_tag(uint64_t epoch) { return uint32_t(epoch % 0xffffffffull) + 1u; }

__device__ __forceinline__ void accumulate8(float* acc, const int4& v) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
    }
}
__device__ __forceinline__ int4 pack8(const float* acc) {
    int4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    return v;
}

// Arrival flags are published by a dedicated warp, not by the transfer warps: a flag needs a system-scope
// release after its row has landed, and that fence waits for remote stores in flight.  A transfer warp only
// appends the flag's address to its ring on this board and reports how many of its bulk stores have COMPLETED
// (cp.async.bulk.wait_group, not .read; up to kStoresInFlight may be pending).  The publisher warp sweeps the
// boards, fences once per sweep and writes the flags of everything that completed since its last sweep.
constexpr int kFlagRing = 32;  // entries per transfer warp
constexpr int kMaxPushWarps = 8;
__device__ __forceinline__ void bulk_wait_depth(int depth) {
    switch (depth) {
        case 4: bulk_wait<4>(); break;
        case 6: bulk_wait<6>(); break;
        case 8: bulk_wait<8>(); break;
        case 12: bulk_wait<12>(); break;
        default: bulk_wait<2>(); break;
    }
}
struct FlagBoard {
    uint32_t* ring[kMaxPushWarps][kFlagRing];
    int completed[kMaxPushWarps];  // transfers whose rows have landed (written by the transfer warp, release)
    int published[kMaxPushWarps];  // transfers whose flags are out (written by the publisher)
    int finished[kMaxPushWarps];   // the transfer warp has no more work
};

struct FlagWriter {  // a transfer warp's end of the board (all lanes hold the same values)
    FlagBoard* board;
    int warp;
    int produced;
    int depth;  // bulk stores that may be pending before the warp waits
    uint64_t timeout_ns;
    // Call right after committing the bulk group of the row that `flag` announces.
    __device__ __forceinline__ void push(uint32_t* flag) {
        const int lane = threadIdx.x & 31;
        if (lane == 0) {
            volatile int* published = board->published + warp;
            if (produced - *published >= kFlagRing) {  // ring full: the publisher is behind (bounded wait)
                const uint64_t start = global_timer_ns();
                while (produced - *published >= kFlagRing && global_timer_ns() - start < timeout_ns) __nanosleep(64);
            }
            board->ring[warp][produced % kFlagRing] = flag;
        }
        ++produced;
        bulk_wait_read<1>();              // the ring stage of the previous row may be refilled
        bulk_wait_depth(depth);           // everything older than the newest `depth` rows has landed
        __syncwarp();                     // other lanes' gate-weight stores are ordered before the hand-over below
        if (lane == 0 && produced > depth) st_release_cta_smem(board->completed + warp, produced - depth);
    }
    __device__ __forceinline__ void finish() {
        bulk_wait<0>();
        __syncwarp();
        if ((threadIdx.x & 31) == 0) {
            st_release_cta_smem(board->completed + warp, produced);
            st_release_cta_smem(board->finished + warp, 1);
        }
    }
};

// The publisher warp of a combine CTA.
__device__ void combine_publish_role(const CombineParams& p, FlagBoard* board) {
    const int lane = threadIdx.x & 31, PW = p.push_warps;
    const uint32_t tag = combine_tag(p.epoch);
    int pub = 0;  // lane w < PW: flags of transfer warp w published so far
    const uint64_t start = global_timer_ns();
    for (;;) {
        const int fin = lane < PW ? ld_acquire_cta_smem(board->finished + lane) : 1;
        const int done = lane < PW ? ld_acquire_cta_smem(board->completed + lane) : 0;
        const unsigned fresh = __ballot_sync(kFull, lane < PW && done > pub);
        if (fresh != 0) {
            fence_acq_rel_sys();  // one release for everything that landed since the last sweep
            for (unsigned left = fresh; left != 0; left &= left - 1) {
                const int w = __ffs(left) - 1;
                const int from = __shfl_sync(kFull, pub, w), to = __shfl_sync(kFull, done, w);
                for (int i = from + lane; i < to; i += 32) st_relaxed_sys_u32(board->ring[w][i % kFlagRing], tag);
            }
            __syncwarp();  // every ring entry has been read before its slot is handed back
            if (lane < PW && done > pub) {
                pub = done;
                *(volatile int*)(board->published + lane) = pub;
            }
        }
        if (__all_sync(kFull, fin != 0 && pub == done)) break;
        if (fresh == 0) {
            __nanosleep(200);
            if (global_timer_ns() - start > 4 * p.c.timeout_ns) {  // transfer warps give up long before this
                if (lane == 0) report(status_of(p.c), kCopyTimeout, 0xfffeu, kTagPush);
                break;
            }
        }
    }
}

// Transfer warps.  Receive rows are visited round-robin over the source ranks (SourceWalk), so at every moment
// the warps of a GPU address all destinations evenly; a row of the expert-major layout yields one transfer per
// local slot.
__device__ void combine_push_role(const CombineParams& p, char* smem, FlagBoard* board) {
    const WindowLayout& L = p.c.layout;
    const int R = L.ranks, K = L.topk, H = L.hidden;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, PW = p.push_warps;
    const int gw = blockIdx.x * PW + warp;
    const StatusRef status = status_of(p.c);
    const int MW = K + 2;
    const uint32_t xb = uint32_t(H) * 2u;
    Ring ring = make_ring(smem, PW, p.stages, xb);
    const int S = p.stages;
    const SourceWalk walk = make_walk(p.recv_rank_prefix, p.c.rank, R);
    // The walk is shared by all transfer warps of the rank: a warp takes the next position from one counter when it
    // needs work (the request for the position after that is already in flight).  Rows differ in how many transfers
    // they need (0 to K local slots), so equal shares of rows leave the warps with the most slots working alone at
    // the end; with a shared position all warps end within one row of each other and rows leave in walk order
    // (measured at 2 GPUs and 4096 tokens per rank: the transfer warps end 8 us earlier).
    int* work = ctrl_words(p.c) + WindowLayout::kWorkCursor;
    int claimed = 0;  // lane 0: the position requested last
    auto request = [&]() {
        if (lane == 0) claimed = atomicAdd(work, 1);
    };
    auto take = [&]() {  // the requested position, on every lane; requests the one after it
        const int v = __shfl_sync(kFull, claimed, 0);
        if (v < walk.items) request();
        return v;
    };
    request();
    const int depth = (p.store_depth == 4 || p.store_depth == 6 || p.store_depth == 8 || p.store_depth == 12) ? p.store_depth : 2;
    FlagWriter flags{board, warp, 0, depth, p.c.timeout_ns};

    if (p.mode == kPushExpandedReduce) {
        // FP32 sum of the row's local slots, one bf16 round, one store per (token, this rank).
        const int vecs = H / 8;
        int q = 0;  // rows sent so far: consecutive rows use consecutive ring stages
        for (;;) {
            const int item = take();
            if (item >= walk.items) break;
            int r;
            const bool live_row = walk.locate(item, r);
            const int* m = p.meta + int64_t(live_row ? r : 0) * MW;
            const int v = (live_row && lane < K) ? m[2 + lane] : -1;
            const unsigned vm = __ballot_sync(kFull, v >= 0 && v < p.capacity);
            const int src = m[0], tok = m[1];
            bool fine = live_row && vm != 0;
            if (fine && (src < 0 || src >= R || tok < 0 || tok >= L.max_tokens || __any_sync(kFull, v >= p.capacity))) {
                if (lane == 0) report(status, kBadMetadata, uint32_t(r), kTagPush);
                fine = false;
            }
            if (!fine) continue;
            char* st = ring.slot(q++);
            // four 16-byte column chunks x two slots per step: eight independent loads per lane in flight
            for (int c0 = lane; c0 < vecs; c0 += 128) {
                float acc[4][8];
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
                unsigned left = vm;
                while (left) {
                    const int k0 = __ffs(left) - 1;
                    left &= left - 1;
                    const int k1 = left ? __ffs(left) - 1 : -1;
                    if (left) left &= left - 1;
                    const int slot0 = __shfl_sync(kFull, v, k0);
                    const int slot1 = __shfl_sync(kFull, v, k1 < 0 ? 0 : k1);
                    const int4* r0 = reinterpret_cast<const int4*>(p.y + int64_t(slot0) * H);
                    const int4* r1 = reinterpret_cast<const int4*>(p.y + int64_t(slot1) * H);
                    int4 d0[4], d1[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (c0 + 32 * u < vecs) {
                            d0[u] = ld_nc_v4(r0 + c0 + 32 * u);
                            if (k1 >= 0) d1[u] = ld_nc_v4(r1 + c0 + 32 * u);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (c0 + 32 * u < vecs) {
                            accumulate8(acc[u], d0[u]);
                            if (k1 >= 0) accumulate8(acc[u], d1[u]);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (c0 + 32 * u < vecs) reinterpret_cast<int4*>(st)[c0 + 32 * u] = pack8(acc[u]);
            }
            fence_proxy_async_smem();
            __syncwarp();
            const int part = L.rank_indexed ? p.c.rank : __ffs(vm) - 1;
            if (lane == 0) bulk_store(ret_row(p.c, src, part, tok), st, xb);
            if (p.w != nullptr && ((vm >> lane) & 1u)) st_relaxed_sys_f32(ret_w_row(p.c, src, tok) + lane, p.w[v]);
            bulk_commit();
            flags.push(ret_flag(p.c, src, part, tok));
        }
        flags.finish();
        return;
    }

    // One bulk load + one bulk store per transfer.  A cursor enumerates the transfers of this warp's rows:
    // compact layout = one per receive row; expert-major layout = one per local slot of the row.
    const bool by_slot = p.mode == kPushExpanded;
    struct Cursor {
        unsigned left;  // choices of the current row that still need a transfer
        unsigned vm;    // all valid choices of the current row
        int r, v, src, tok, k;
    };
    // The loads run ahead of the stores over the same sequence of rows: the leading cursor takes positions from the
    // shared counter and queues the live ones (lane n % 32 keeps the n-th), the trailing cursor reads them back.
    int queued = 0, q_head = 0, q_tail = 0;
    auto next = [&](Cursor& c, bool leading) {
        while (c.left == 0) {
            int r;
            if (leading) {
                const int item = take();
                if (item >= walk.items) return false;
                if (!walk.locate(item, r)) continue;
                if (lane == (q_head & 31)) queued = r;
                ++q_head;
            } else {
                if (q_tail == q_head) return false;
                r = __shfl_sync(kFull, queued, q_tail & 31);
                ++q_tail;
            }
            const int* m = p.meta + int64_t(r) * MW;
            c.r = r;
            c.src = m[0];
            c.tok = m[1];
            c.v = lane < K ? m[2 + lane] : -1;
            c.vm = __ballot_sync(kFull, c.v >= 0);
            const bool bad_slot = __any_sync(kFull, by_slot && c.v >= p.capacity);
            if (c.src < 0 || c.src >= R || c.tok < 0 || c.tok >= L.max_tokens || bad_slot) {
                if (lane == 0) report(status, kBadMetadata, uint32_t(r), kTagPush);
                c.vm = 0;
            }
            c.left = by_slot ? c.vm : (c.vm & (0u - c.vm));  // compact: the first valid choice names the partition
        }
        c.k = __ffs(c.left) - 1;
        c.left &= c.left - 1;
        return true;
    };
    const uint64_t once = l2_evict_first_policy();  // expert rows are read exactly once: keep L2 for the return rows
    auto issue = [&](const Cursor& c, int q) {
        const int y_row = by_slot ? __shfl_sync(kFull, c.v, c.k) : c.r;
        if (lane == 0) {
            mbar_expect_tx(ring.bar(q), xb);
            bulk_load_hint(ring.slot(q), p.y + int64_t(y_row) * H, xb, ring.bar(q), once);
        }
    };
    Cursor ahead{0u, 0u, 0, -1, 0, 0, 0}, now{0u, 0u, 0, -1, 0, 0, 0};
    int issued = 0;
    bool more = true;
    while (issued < S - 1 && (more = next(ahead, true))) issue(ahead, issued++);
    for (int q = 0; next(now, false); ++q) {
        if (!ring.wait(q, p.c.timeout_ns)) {
            if (lane == 0) report(status, kCopyTimeout, uint32_t(gw), kTagPush);
            break;
        }
        const int part = by_slot ? now.k : (L.rank_indexed ? p.c.rank : now.k);
        if (lane == 0) bulk_store(ret_row(p.c, now.src, part, now.tok), ring.slot(q), xb);
        if (p.w != nullptr) {
            if (by_slot) {
                const int slot = __shfl_sync(kFull, now.v, now.k);
                if (lane == 0) st_relaxed_sys_f32(ret_w_row(p.c, now.src, now.tok) + now.k, p.w[slot]);
            } else if ((now.vm >> lane) & 1u) {
                st_relaxed_sys_f32(ret_w_row(p.c, now.src, now.tok) + lane, p.w[int64_t(now.r) * K + lane]);
            }
        }
        bulk_commit();
        flags.push(ret_flag(p.c, now.src, part, now.tok));
        if (more && (more = next(ahead, true))) issue(ahead, issued++);
    }
    flags.finish();
}

// Which return partitions hold a row for source token `t`, as a mask over the lanes (choices) that name them;
// `valid` is the lane's own choice.  One partition per valid choice, or one per destination rank (named by
// the rank's first choice).
__device__ __forceinline__ unsigned expected_parts(const int64_t* topk, int t, int K, int E, int Le, bool sum_all_choices, bool& valid,
                                                   int& dest) {
    const int lane = threadIdx.x & 31;
    const int64_t e = lane < K ? topk[int64_t(t) * K + lane] : -1;
    valid = e >= 0 && e < E;
    dest = valid ? int(e) / Le : -1;
    const unsigned vmask = __ballot_sync(kFull, valid);
    if (sum_all_choices) return vmask;
    bool leader = false;
    if (valid) {
        const unsigned same = __match_any_sync(vmask, dest);
        leader = lane == __ffs(same) - 1;
    }
    return __ballot_sync(kFull, leader);
}

// FP32 sum of the partitions in `parts` for the 16-byte column chunks `first`, `first + step`, ... of token t.
// All partitions of a chunk are loaded before any is added, two chunks at a time.
__device__ __forceinline__ void reduce_columns(const CommonParams& c, int t, unsigned parts, int my_part, const __nv_bfloat16* bias,
                                               __nv_bfloat16* out, int first_base, int step, uint64_t once) {
    const WindowLayout& L = c.layout;
    const int H = L.hidden, lane = threadIdx.x & 31;
    const int vecs = H / 8;
    const int64_t part_stride = L.max_tokens * int64_t(H) * 2;
    const char* row0 = window(c, c.rank) + L.ret_offset + int64_t(t) * H * 2;
    // `base` is the same for every lane of the warp (the loop holds warp shuffles); lanes past the row's end idle
    for (int base = first_base; base < vecs; base += 2 * step) {
        const int col = base + lane;
        const bool one = col < vecs, two = col + step < vecs;
        float a0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        float a1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        unsigned left = parts;
        while (left) {
            int part[8];
            int4 d0[8], d1[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int k = left ? __ffs(left) - 1 : -1;
                if (left) left &= left - 1;
                part[j] = __shfl_sync(kFull, my_part, k < 0 ? 0 : k);
                if (k < 0) part[j] = -1;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (part[j] >= 0) {
                    const int4* src = reinterpret_cast<const int4*>(row0 + part[j] * part_stride);
                    if (one) d0[j] = ld_cg_v4_hint(src + col, once);
                    if (two) d1[j] = ld_cg_v4_hint(src + col + step, once);
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (part[j] >= 0) {
                    if (one) accumulate8(a0, d0[j]);
                    if (two) accumulate8(a1, d1[j]);
                }
            }
        }
        if (bias != nullptr) {
            const int4* b = reinterpret_cast<const int4*>(bias + int64_t(t) * H);
            if (one) accumulate8(a0, ld_nc_v4(b + col));
            if (two) accumulate8(a1, ld_nc_v4(b + col + step));
        }
        int4* o = reinterpret_cast<int4*>(out + int64_t(t) * H);
        if (one) st_v4_hint(o + col, pack8(a0), once);
        if (two) st_v4_hint(o + col + step, pack8(a1), once);
    }
}

constexpr int kReduceFlowWords = 2 + 2 * (kCombineThreads / 32 + 1);

// Reduce warps of the combine kernel.  They form groups of `reduce_group` warps; a group sums ONE source token at a
// time, each lane its own column chunks.  The group's first warp waits (bounded) until every partition the token
// expects carries this combine's tag and releases the others through the group's named barrier.
//
// How long one token takes decides how long the kernel runs after the last row has landed: under the load of the
// transfers a group of two warps needs ~30 us per token (seven dependent batches of loads at ~4 us each), five warps
// ~13 us, all ten ~9 us - but larger groups hold fewer tokens at a time and fall behind the arrivals, and handing only
// the last tokens of a CTA to all of its warps measured slower as well (they are summed one after the other).
//
// `flow` is a small shared array: [0] the CTA's abort word (sticky), then two go/stop words per group.  The warp that waited writes "go" or "stop" into the word of the barrier's
// parity BEFORE the barrier and everybody reads it AFTER the barrier, so all warps of a barrier take the same branch
// (reading the sticky abort word instead would let two warps of one barrier see different values and strand one of
// them at the next barrier, which has no time limit).
__device__ void combine_reduce_role(const CombineParams& p, int* flow) {
    int* abort_word = flow;
    const WindowLayout& L = p.c.layout;
    const int K = L.topk, Le = L.local_experts, E = int(L.num_experts);
    const int lane = threadIdx.x & 31;
    const int RW = (blockDim.x >> 5) - p.push_warps - 1;  // one warp publishes flags
    const int rwarp = (threadIdx.x >> 5) - p.push_warps - 1;
    const int G = p.reduce_group < 1 ? 1 : (p.reduce_group > RW ? RW : p.reduce_group);
    const int groups = RW / G, g = rwarp / G, wi = rwarp % G;
    const StatusRef status = status_of(p.c);
    const uint32_t tag = combine_tag(p.epoch);
    const uint32_t* flag_base = reinterpret_cast<const uint32_t*>(window(p.c, p.c.rank) + L.ret_flag_offset);
    const float* ret_w = reinterpret_cast<const float*>(window(p.c, p.c.rank) + L.ret_w_offset);
    // returned rows are read once and the result is written once: both leave L2 first
    const uint64_t once = l2_evict_first_policy();
    unsigned waited = 0, worked = 0, longest = 0, summed = 0;  // nanoseconds (a kernel runs far below four seconds)
    unsigned long long longest_at = 0, last_seen = 0;

    // One warp waits for the token's rows (bounded); on a timeout it reports and raises the CTA's abort word.
    auto await_rows = [&](int t, unsigned parts, int my_part) -> bool {
        const bool mine = (parts >> lane) & 1u;
        const uint32_t* flag = flag_base + int64_t(mine ? my_part : 0) * L.max_tokens + t;
        const uint64_t start = global_timer_ns();
        uint32_t spins = 0;
        bool arrived = false;
        for (;;) {
            const bool here = !mine || ld_relaxed_sys_u32(flag) == tag;
            arrived = __all_sync(kFull, here);
            if (arrived) break;
            __nanosleep(200);
            if ((++spins & 15u) == 0u && __any_sync(kFull, global_timer_ns() - start > p.c.timeout_ns)) break;
        }
        // the polls were relaxed; one acquiring load of each flag orders the rows behind them
        if (arrived && mine) (void)ld_acquire_sys_u32(flag);
        __syncwarp();
        if (!arrived && lane == 0) {
            report(status, kBarrierTimeout, uint32_t(t), kTagReduce);
            *(volatile int*)abort_word = 1;  // a peer never delivered: stop reducing, the host reports the status
        }
        return arrived;
    };
    auto sum_token = [&](int t, unsigned parts, int my_part, bool valid, bool first_warp, int first_base, int step, uint64_t t_wait) {
        const uint64_t t_work = p.trace != nullptr ? global_timer_ns() : 0;
        reduce_columns(p.c, t, parts, my_part, p.bias, p.out, first_base, step, once);
        if (first_warp && p.w_out != nullptr && lane < K) p.w_out[int64_t(t) * K + lane] = valid ? __ldcg(ret_w + int64_t(t) * K + lane) : 0.f;
        if (p.trace != nullptr) {
            const uint64_t t_done = global_timer_ns();
            waited += unsigned(t_work - t_wait);
            worked += unsigned(t_done - t_work);
            if (unsigned(t_done - t_work) > longest) {
                longest = unsigned(t_done - t_work);
                longest_at = t_work;
            }
            last_seen = t_work;
            ++summed;
        }
    };

    // warps that do not fill a group sit out
    if (g < groups) {
        int* go = flow + 2 + 2 * g;
        unsigned syncs = 0;
        for (int t = blockIdx.x * groups + g; t < p.tokens; t += gridDim.x * groups) {
            bool valid;
            int dest;
            const unsigned parts = expected_parts(p.topk, t, K, E, Le, p.sum_all_choices != 0, valid, dest);
            const int my_part = L.rank_indexed ? dest : lane;
            const uint64_t t_wait = p.trace != nullptr ? global_timer_ns() : 0;
            if (parts != 0) {
                bool ok = true;
                if (wi == 0) {
                    ok = !*(volatile int*)abort_word && await_rows(t, parts, my_part);
                    if (G > 1 && lane == 0) *(volatile int*)(go + (syncs & 1u)) = ok;
                }
                if (G > 1) {
                    // named barrier 1 + g: this group's reduce warps only
                    asm volatile("bar.sync %0, %1;" ::"r"(1 + g), "r"(G * 32) : "memory");
                    ok = *(volatile int*)(go + (syncs & 1u)) != 0;
                    ++syncs;
                }
                if (!ok) break;
            }
            sum_token(t, parts, my_part, valid, wi == 0, wi * 32, G * 32, t_wait);
        }
    }
    if (p.trace != nullptr && (rwarp % G) == 0 && lane == 0) {
        atomicAdd(p.trace + 4, (unsigned long long)waited);
        atomicAdd(p.trace + 5, (unsigned long long)worked);
        atomicAdd(p.trace + 6, (unsigned long long)summed);
        const unsigned long long t0 = *(volatile unsigned long long*)p.trace;
        atomicMax(p.trace + 7, ((unsigned long long)longest << 32) | (unsigned long long)unsigned(longest_at - t0));
        atomicMax(p.trace + 8, last_seen);
    }
}

// Bounded mbarrier wait of the reduce pipeline: also gives up as soon as the CTA's abort word is raised.
__device__ __forceinline__ bool mbar_wait_or_abort(uint64_t* bar, uint32_t parity, uint64_t timeout_ns, const int* abort_word) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63u) == 0u && (*(volatile const int*)abort_word != 0 || global_timer_ns() - start > timeout_ns)) return false;
    }
    return true;
}

// Where the reduce pipeline's stages start in dynamic shared memory (behind the transfer rings and the flag board).
__device__ __forceinline__ char* reduce_area(const CombineParams& p, char* smem) {
    const int64_t ring_end = (align_up(int64_t(p.c.layout.hidden) * 2, 128) + 8) * int64_t(p.push_warps) * p.stages;
    const uintptr_t board = (reinterpret_cast<uintptr_t>(smem + ring_end) + 15) & ~uintptr_t(15);
    return reinterpret_cast<char*>((board + sizeof(FlagBoard) + 127) & ~uintptr_t(127));
}

// The source-side sum fed through shared memory.  The CTA sums ONE of its tokens at a time: the first reduce warp
// (the loader) waits for the token's arrival flags and bulk-loads `reduce_chunk_bytes` of every expected partition
// row into the next free stage of a small ring; the other reduce warps wait on the stage's mbarrier, add the rows
// in FP32 in ascending partition order straight from shared memory, add the bias, round once and store.  A bulk load
// keeps no registers busy, so all partitions of a chunk are in flight at once and several chunks ahead: what is left
// of the kernel after the last row has landed is one load latency and a sum from shared memory, where the register
// path needs seven dependent batches of loads per token.
__device__ void combine_reduce_smem_role(const CombineParams& p, int* flow, char* area) {
    int* abort_word = flow;
    const WindowLayout& L = p.c.layout;
    const int K = L.topk, Le = L.local_experts, E = int(L.num_experts), H = L.hidden, P = L.ret_parts;
    const int lane = threadIdx.x & 31;
    const int RW = (blockDim.x >> 5) - p.push_warps - 1;
    const int rwarp = (threadIdx.x >> 5) - p.push_warps - 1;
    const int CW = RW - 1;  // consumer warps
    const int NS = p.reduce_stages, cw = p.reduce_chunk_bytes, xb = H * 2;
    const int nc = (xb + cw - 1) / cw;
    uint64_t* full = reinterpret_cast<uint64_t*>(area + int64_t(NS) * P * cw);
    uint64_t* empty = full + NS;
    const StatusRef status = status_of(p.c);
    const uint32_t tag = combine_tag(p.epoch);
    const int n_tok = p.tokens > int(blockIdx.x) ? (p.tokens - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;
    const int units = n_tok * nc;
    const uint64_t once = l2_evict_first_policy();

    if (rwarp == 0) {
        // ---- loader
        const uint32_t* flag_base = reinterpret_cast<const uint32_t*>(window(p.c, p.c.rank) + L.ret_flag_offset);
        const float* ret_w = reinterpret_cast<const float*>(window(p.c, p.c.rank) + L.ret_w_offset);
        unsigned parts = 0;
        int my_part = 0;
        for (int u = 0; u < units; ++u) {
            const int c = u % nc, t = int(blockIdx.x) + (u / nc) * int(gridDim.x);
            const int s = u % NS, n = u / NS;
            if (c == 0) {
                bool valid;
                int dest;
                parts = expected_parts(p.topk, t, K, E, Le, p.sum_all_choices != 0, valid, dest);
                my_part = L.rank_indexed ? dest : lane;
                if (parts != 0) {
                    const bool mine = (parts >> lane) & 1u;
                    const uint32_t* flag = flag_base + int64_t(mine ? my_part : 0) * L.max_tokens + t;
                    const uint64_t start = global_timer_ns();
                    uint32_t spins = 0;
                    bool arrived = false;
                    for (;;) {
                        const bool here = !mine || ld_relaxed_sys_u32(flag) == tag;
                        arrived = __all_sync(kFull, here);
                        if (arrived) break;
                        __nanosleep(100);
                        if ((++spins & 15u) == 0u &&
                            __any_sync(kFull, *(volatile int*)abort_word != 0 || global_timer_ns() - start > p.c.timeout_ns))
                            break;
                    }
                    // the polls were relaxed; one acquiring load of each flag orders the rows behind them, and the
                    // proxy fence orders the bulk loads below behind that
                    if (arrived && mine) (void)ld_acquire_sys_u32(flag);
                    fence_proxy_async();
                    __syncwarp();
                    if (!arrived) {
                        if (lane == 0) {
                            report(status, kBarrierTimeout, uint32_t(t), kTagReduce);
                            *(volatile int*)abort_word = 1;  // a peer never delivered: the consumers stop at their next wait
                        }
                        break;
                    }
                }
                if (p.w_out != nullptr && lane < K) p.w_out[int64_t(t) * K + lane] = valid ? __ldcg(ret_w + int64_t(t) * K + lane) : 0.f;
            }
            if (n >= 1) {
                // the stage is free once every consumer warp has read its previous contents
                bool ok = mbar_wait_or_abort(empty + s, uint32_t(n - 1) & 1u, p.c.timeout_ns, abort_word);
                ok = __all_sync(kFull, ok);
                if (!ok) {
                    if (lane == 0 && *(volatile int*)abort_word == 0) {
                        report(status, kCopyTimeout, uint32_t(t), kTagReduce);
                        *(volatile int*)abort_word = 1;
                    }
                    break;
                }
            }
            const int bytes = min(cw, xb - c * cw);
            if (lane == 0) mbar_expect_tx(full + s, uint32_t(__popc(parts) * bytes));
            __syncwarp();
            if ((parts >> lane) & 1u) {
                const int j = __popc(parts & lanemask_lt());
                bulk_load_hint(area + (int64_t(s) * P + j) * cw, ret_row(p.c, p.c.rank, my_part, t) + int64_t(c) * cw, uint32_t(bytes),
                               full + s, once);
            }
        }
        return;
    }

    // ---- consumers
    const int cwarp = rwarp - 1;
    unsigned parts = 0;
    unsigned waited = 0, worked = 0, longest = 0, summed = 0;  // nanoseconds
    unsigned long long longest_at = 0, last_seen = 0;
    for (int u = 0; u < units; ++u) {
        const int c = u % nc, t = int(blockIdx.x) + (u / nc) * int(gridDim.x);
        const int s = u % NS, n = u / NS;
        if (c == 0) {
            bool valid;
            int dest;
            parts = expected_parts(p.topk, t, K, E, Le, p.sum_all_choices != 0, valid, dest);
        }
        const uint64_t t_wait = p.trace != nullptr ? global_timer_ns() : 0;
        {
            bool ok = mbar_wait_or_abort(full + s, uint32_t(n) & 1u, p.c.timeout_ns, abort_word);
            ok = __all_sync(kFull, ok);
            if (!ok) {
                if (lane == 0 && *(volatile int*)abort_word == 0) {
                    report(status, kCopyTimeout, uint32_t(t), kTagReduce);
                    *(volatile int*)abort_word = 1;
                }
                break;
            }
        }
        const uint64_t t_work = p.trace != nullptr ? global_timer_ns() : 0;
        const int np = __popc(parts);
        const int bytes = min(cw, xb - c * cw);
        const char* rows = area + int64_t(s) * P * cw;
        for (int v = cwarp * 32 + lane; v * 16 < bytes; v += CW * 32) {
            float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
            for (int j = 0; j < np; ++j) accumulate8(a, *reinterpret_cast<const int4*>(rows + int64_t(j) * cw + v * 16));
            const int64_t at = (int64_t(t) * xb + int64_t(c) * cw) / 16 + v;  // 16-byte units from the start of the output
            if (p.bias != nullptr) accumulate8(a, ld_nc_v4(reinterpret_cast<const int4*>(p.bias) + at));
            st_v4_hint(reinterpret_cast<int4*>(p.out) + at, pack8(a), once);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
        if (p.trace != nullptr) {
            const uint64_t t_done = global_timer_ns();
            waited += unsigned(t_work - t_wait);
            worked += unsigned(t_done - t_work);
            if (unsigned(t_done - t_work) > longest) {
                longest = unsigned(t_done - t_work);
                longest_at = t_work;
            }
            last_seen = t_work;
            summed += c == 0 ? 1u : 0u;
        }
    }
    if (p.trace != nullptr && cwarp == 0 && lane == 0) {
        atomicAdd(p.trace + 4, (unsigned long long)waited);
        atomicAdd(p.trace + 5, (unsigned long long)worked);
        atomicAdd(p.trace + 6, (unsigned long long)summed);
        const unsigned long long t0 = *(volatile unsigned long long*)p.trace;
        atomicMax(p.trace + 7, ((unsigned long long)longest << 32) | (unsigned long long)unsigned(longest_at - t0));
        atomicMax(p.trace + 8, last_seen);
    }
}

__device__ void combine_body(const CombineParams& p) {
    extern __shared__ __align__(128) char s_ring[];
    __shared__ int s_enter;
    __shared__ int s_flow[kReduceFlowWords];  // see combine_reduce_role
    const WindowLayout& L = p.c.layout;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const StatusRef status = status_of(p.c);
    int* ctrl = ctrl_words(p.c);
    // the flag board sits behind the transfer rings (plan_ring leaves room for it)
    FlagBoard* board = reinterpret_cast<FlagBoard*>(
        (reinterpret_cast<uintptr_t>(s_ring + (align_up(int64_t(L.hidden) * 2, 128) + 8) * int64_t(p.push_warps) * p.stages) + 15) & ~uintptr_t(15));
    if (threadIdx.x == 0) {
        s_enter = 1;
        if (p.reduce_stages >= 2) {
            // full: the loader's arrival plus the bytes of its bulk loads; empty: one arrival per consumer warp
            char* area = reduce_area(p, s_ring);
            uint64_t* full = reinterpret_cast<uint64_t*>(area + int64_t(p.reduce_stages) * L.ret_parts * p.reduce_chunk_bytes);
            const int consumers = int(blockDim.x >> 5) - p.push_warps - 2;
            for (int s = 0; s < p.reduce_stages; ++s) {
                mbar_init(full + s, 1);
                mbar_init(full + p.reduce_stages + s, uint32_t(consumers));
            }
            mbar_init_fence();
            fence_proxy_async_smem();
        }
    }
    if (threadIdx.x < kReduceFlowWords) s_flow[threadIdx.x] = 0;
    if (threadIdx.x < kMaxPushWarps) board->completed[threadIdx.x] = board->published[threadIdx.x] = board->finished[threadIdx.x] = 0;
    __syncthreads();
    if (p.wait_epoch != 0) {
        // Every peer has finished reading what the previous combine left in its return area.
        if (warp == 0) {
            const bool ok = peer_wait_warp(p.c.peers, p.c.rank, L.ranks, L.signal_offset, p.wait_epoch, p.c.timeout_ns, status, kTagPush);
            if (lane == 0) s_enter = ok;
        }
        __syncthreads();
    }
    if (p.trace != nullptr && threadIdx.x == 0) atomicMin(p.trace, global_timer_ns());
    if (s_enter) {
        const int role = warp < p.push_warps ? 1 : warp == p.push_warps ? 2 : 3;
        if (role == 1)
            combine_push_role(p, s_ring, board);
        else if (role == 2)
            combine_publish_role(p, board);
        else if (p.reduce_stages >= 2)
            combine_reduce_smem_role(p, s_flow, reduce_area(p, s_ring));
        else
            combine_reduce_role(p, s_flow);
        if (p.trace != nullptr && lane == 0) atomicMax(p.trace + role, global_timer_ns());
    }
    // The last block out tells every peer that this rank is done with the combine (nobody waits here).  Rows and
    // flags are out already (completed bulk groups, the publishers' fences); the ticket orders this block's reads of
    // the return area before the signal that lets peers overwrite it.
    if (!take_last_ticket(ctrl + WindowLayout::kTicketCombine)) return;
    if (threadIdx.x == 0) {
        ctrl[WindowLayout::kTicketCombine] = 0;
        ctrl[WindowLayout::kWorkCursor] = 0;  // every transfer warp of the rank is done: the next combine starts its walk at 0
    }
    __threadfence_system();
    __syncthreads();
    if (warp == 0) peer_signal_warp(p.c.peers, p.c.rank, L.ranks, L.signal_offset, p.epoch);
}

// ------------------------------------------------------------------------------------------
// reduce alone: source-side sum of rows that another kernel pushed and a peer barrier made visible.
// ------------------------------------------------------------------------------------------
__device__ void reduce_body(const ReduceParams& p) {
    const WindowLayout& L = p.c.layout;
    const int K = L.topk, Le = L.local_experts, E = int(L.num_experts);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    const int gw = blockIdx.x * wpb + warp, GW = gridDim.x * wpb;
    const float* ret_w = reinterpret_cast<const float*>(window(p.c, p.c.rank) + L.ret_w_offset);
    for (int t = gw; t < p.tokens; t += GW) {
        bool valid;
        int dest;
        const unsigned parts = expected_parts(p.topk, t, K, E, Le, p.sum_all_choices != 0, valid, dest);
        reduce_columns(p.c, t, parts, L.rank_indexed ? dest : lane, p.bias, p.out, 0, 32, l2_evict_first_policy());
        if (p.w_out != nullptr && lane < K) p.w_out[int64_t(t) * K + lane] = valid ? __ldcg(ret_w + int64_t(t) * K + lane) : 0.f;
    }
}

// ------------------------------------------------------------------------------------------
// local combine (single-rank group): sum a row's expert outputs into its source token.
// ------------------------------------------------------------------------------------------
__device__ void local_combine_body(const LocalCombineParams& p) {
    const WindowLayout& L = p.c.layout;
    const int K = L.topk, H = L.hidden;
    const int E = int(L.num_experts);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    const int gw = blockIdx.x * wpb + warp, GW = gridDim.x * wpb;
    const int MW = K + 2, vecs = H / 8;
    const StatusRef status = status_of(p.c);
    for (int r = gw; r < p.rows; r += GW) {
        const int* m = p.meta + int64_t(r) * MW;
        const int tok = m[1];
        if (m[0] != p.c.rank || tok < 0 || tok >= p.tokens) {
            if (lane == 0) report(status, kBadMetadata, uint32_t(r), kTagReduce);
            continue;
        }
        const int v = lane < K ? m[2 + lane] : -1;
        const unsigned vm = __ballot_sync(kFull, p.expand ? (v >= 0 && v < p.capacity) : v >= 0);
        if (vm == 0) continue;
        const int4* bias = p.bias != nullptr ? reinterpret_cast<const int4*>(p.bias + int64_t(tok) * H) : nullptr;
        int4* out = reinterpret_cast<int4*>(p.out + int64_t(tok) * H);
        for (int c = lane; c < vecs; c += 64) {
            const bool two = c + 32 < vecs;
            float a0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            float a1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (p.expand) {
                unsigned left = vm;
                while (left) {
                    int k[4];
                    int4 d0[4], d1[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        k[j] = left ? __ffs(left) - 1 : -1;
                        if (left) left &= left - 1;
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int slot = __shfl_sync(kFull, v, k[j] < 0 ? 0 : k[j]);
                        if (k[j] >= 0) {
                            const int4* src = reinterpret_cast<const int4*>(p.y + int64_t(slot) * H);
                            d0[j] = ld_nc_v4(src + c);
                            if (two) d1[j] = ld_nc_v4(src + c + 32);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (k[j] >= 0) {
                            accumulate8(a0, d0[j]);
                            if (two) accumulate8(a1, d1[j]);
                        }
                    }
                }
                if (p.round_partial) {
                    const int4 r0 = pack8(a0), r1 = pack8(a1);
#pragma unroll
                    for (int j = 0; j < 8; ++j) a0[j] = a1[j] = 0.f;
                    accumulate8(a0, r0);
                    accumulate8(a1, r1);
                }
            } else {
                const int4* src = reinterpret_cast<const int4*>(p.y + int64_t(r) * H);
                accumulate8(a0, ld_nc_v4(src + c));
                if (two) accumulate8(a1, ld_nc_v4(src + c + 32));
            }
            if (bias != nullptr) {
                accumulate8(a0, ld_nc_v4(bias + c));
                if (two) accumulate8(a1, ld_nc_v4(bias + c + 32));
            }
            out[c] = pack8(a0);
            if (two) out[c + 32] = pack8(a1);
        }
        if (p.w_out != nullptr && lane < K) {
            float wv = 0.f;
            if ((vm >> lane) & 1u) wv = p.expand ? p.w[v] : p.w[int64_t(r) * K + lane];
            p.w_out[int64_t(tok) * K + lane] = wv;
        }
    }
    // tokens without any valid choice have no receive row: result = bias (or zero), weights = 0
    for (int t = gw; t < p.tokens; t += GW) {
        const int64_t e = lane < K ? p.topk[int64_t(t) * K + lane] : -1;
        if (__ballot_sync(kFull, e >= 0 && e < E) != 0) continue;
        int4* out = reinterpret_cast<int4*>(p.out + int64_t(t) * H);
        const int4* bias = p.bias != nullptr ? reinterpret_cast<const int4*>(p.bias + int64_t(t) * H) : nullptr;
        for (int c = lane; c < vecs; c += 32) out[c] = bias != nullptr ? ld_nc_v4(bias + c) : make_int4(0, 0, 0, 0);
        if (p.w_out != nullptr && lane < K) p.w_out[int64_t(t) * K + lane] = 0.f;
    }
}

__device__ void barrier_body(const BarrierParams& p) {
    if (p.signal_only) {
        __threadfence_system();
        peer_signal_warp(p.c.peers, p.c.rank, p.c.layout.ranks, p.c.layout.signal_offset, p.epoch);
        return;
    }
    peer_barrier_warp(p.c.peers, p.c.rank, p.c.layout.ranks, p.c.layout.signal_offset, p.epoch, p.c.timeout_ns, status_of(p.c),
                      kTagBarrier);
}

// Test utility: holds a stream until a word in pinned host memory becomes non-zero (bounded; gate[1] = 1 when the wait
// ran out).  The poll is a system-scope load: it must not be served from a cache on the GPU.
// Lets a test keep one rank's kernel pending at a chosen point while the other ranks run on.
__global__ void gate_kernel(volatile int* gate, uint64_t timeout_ns) {
    const uint64_t start = global_timer_ns();
    while (ld_relaxed_sys(const_cast<const int*>(gate)) == 0) {
        __nanosleep(500);
        if (global_timer_ns() - start > timeout_ns) {
            gate[1] = 1;
            break;
        }
    }
}

// ---------------------------------------------------------------- wrappers
#define NEP_KERNEL_PAIR(name, Params, threads)                                                                  \
    __global__ void __launch_bounds__(threads) name##_kernel(const __grid_constant__ Params p) { name##_body(p); } \
    __global__ void __launch_bounds__(threads) name##_multi_kernel(const Params* all) { name##_body(all[blockIdx.y]); }

__global__ void __launch_bounds__(kStageThreads) stage_kernel(const __grid_constant__ StageParams p) { stage_body(p); }
__global__ void __launch_bounds__(kStageThreads) stage_multi_kernel(const StageParams* all) { stage_body(all[blockIdx.y]); }
NEP_KERNEL_PAIR(plan, PlanParams, kPlanThreads)
NEP_KERNEL_PAIR(pull, PullParams, 256)
__global__ void __launch_bounds__(kCombineThreads, 1) combine_kernel(const __grid_constant__ CombineParams p) { combine_body(p); }
__global__ void __launch_bounds__(kCombineThreads, 1) combine_multi_kernel(const CombineParams* all) { combine_body(all[blockIdx.y]); }
NEP_KERNEL_PAIR(reduce, ReduceParams, kReduceThreads)
NEP_KERNEL_PAIR(barrier, BarrierParams, 32)
NEP_KERNEL_PAIR(local_combine, LocalCombineParams, kReduceThreads)

// Fresh dispatch of a small call in ONE cooperative launch: stage (count exchange, peer barrier, prefixes, mailbox),
// plan, pull.  Outputs are sized by the caller at an upper bound and trimmed on the host once N and C are known, so
// the host's wait for the mailbox runs beside the kernel instead of between two launches.
__device__ void fused_fresh_dispatch_body(const StageParams& sp, const PlanParams& lp, const PullParams& pp) {
    if (!stage_body(sp)) return;
    plan_body(lp);
    // every block of this rank has planned its chunks before any row is pulled
    int* ctrl = ctrl_words(sp.c);
    if (take_last_ticket(ctrl + WindowLayout::kTicketPlan)) {
        if (threadIdx.x == 0) {
            ctrl[WindowLayout::kTicketPlan] = 0;
            publish_go(ctrl, sp.epoch, true, WindowLayout::kGoWordPlan);
        }
    } else if (!wait_go(ctrl, sp.epoch, sp.c.timeout_ns, status_of(sp.c), kTagPlan, WindowLayout::kGoWordPlan)) {
        return;
    }
    __syncthreads();
    fence_proxy_async();
    pull_body(pp);
}
__global__ void __launch_bounds__(256) fused_fresh_dispatch_kernel(const __grid_constant__ StageParams sp, const __grid_constant__ PlanParams lp,
                                                                   const __grid_constant__ PullParams pp) {
    fused_fresh_dispatch_body(sp, lp, pp);
}
__global__ void __launch_bounds__(256) fused_fresh_dispatch_multi_kernel(const StageParams* sp, const PlanParams* lp, const PullParams* pp) {
    fused_fresh_dispatch_body(sp[blockIdx.y], lp[blockIdx.y], pp[blockIdx.y]);
}

// stage + peer barrier + pull in one cooperative launch (cached dispatch, small calls)
__global__ void __launch_bounds__(256) fused_cached_dispatch_kernel(const __grid_constant__ StageParams sp, const __grid_constant__ PullParams pp) {
    if (!stage_body(sp)) return;
    fence_proxy_async();
    pull_body(pp);
}
__global__ void __launch_bounds__(256) fused_cached_dispatch_multi_kernel(const StageParams* sp, const PullParams* pp) {
    if (!stage_body(sp[blockIdx.y])) return;
    fence_proxy_async();
    pull_body(pp[blockIdx.y]);
}

template <typename Params>
cudaError_t launch_pair(void (*single)(const Params), void (*multi)(const Params*), const Params* params, LaunchShape shape, int threads,
                        size_t smem, cudaStream_t stream) {
    if (smem > 48 * 1024) {
        // Raise the kernel's dynamic shared-memory limit once per (kernel, device) and only when it grows.
        static thread_local size_t granted[2][64] = {};
        int device = 0;
        cudaGetDevice(&device);
        size_t& have = granted[shape.ranks_y > 1 ? 1 : 0][device & 63];
        if (smem > have) {
            cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(shape.ranks_y > 1 ? (const void*)multi : (const void*)single),
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
            if (e != cudaSuccess) return e;
            have = smem;
        }
    }
    const dim3 grid(shape.grid_x, shape.ranks_y > 1 ? shape.ranks_y : 1);
    if (shape.ranks_y > 1)
        multi<<<grid, threads, smem, stream>>>(params);
    else
        single<<<grid, threads, smem, stream>>>(*params);
    return cudaGetLastError();
}

}  // namespace

int stage_smem_bytes(const WindowLayout& l) { return int((l.ranks + l.num_experts) * 4); }
int plan_smem_bytes(const WindowLayout& l) { return (kPlanThreads / 32) * 32 * l.topk * 4; }

RingPlan plan_ring(int64_t row_bytes, int max_smem_bytes) {
    // smem = warps * stages * (row pitch + one mbarrier) + zero buffer + alignment slack + static smem.
    // The software pipeline needs at least two stages; a row that does not fit twice is rejected by
    // the caller (warps == 0).
    const int64_t pitch = align_up(row_bytes, 128);
    const int64_t fixed = kZeroBytes + 256 + 256;
    RingPlan r{};
    r.stages = 3;
    int warps = int((int64_t(max_smem_bytes) - fixed) / ((pitch + 8) * r.stages));
    // Under a small budget two warps with two stages beat one warp with three: the same number of
    // loads in flight, twice the instruction issue.
    const int warps2 = int((int64_t(max_smem_bytes) - fixed) / ((pitch + 8) * 2));
    if (warps < 2 && warps2 > warps) {
        r.stages = 2;
        warps = warps2;
    }
    if (warps < 1) warps = 0;
    r.warps = warps > 8 ? 8 : warps;
    r.smem_bytes = size_t(r.warps) * r.stages * (pitch + 8) + kZeroBytes + 256;
    return r;
}

CombinePlan plan_combine(int64_t row_bytes, int parts, int max_smem_bytes, int reduce_stages, int reduce_chunk_bytes) {
    // smem = transfer rings (warps x stages x (row pitch + mbarrier)) + flag board + reduce pipeline
    // (stages x parts x chunk + two mbarriers per stage) + alignment slack + static smem.
    CombinePlan c{};
    const int64_t pitch = align_up(row_bytes, 128);
    const int64_t fixed = int64_t(sizeof(FlagBoard)) + 16 + 128 + 512;
    int64_t chunk = 0;
    if (reduce_stages >= 2) {
        // about half of shared memory for the pipeline unless the caller names a chunk; whole rows when they fit
        chunk = reduce_chunk_bytes > 0 ? align_up(reduce_chunk_bytes, 128) : (int64_t(max_smem_bytes) / 2 / reduce_stages / parts) / 128 * 128;
        chunk = std::min<int64_t>(chunk, pitch);
    }
    // transfer warps the rings would get without a pipeline: an automatic chunk shrinks rather than take the second one
    const int64_t alone = std::min<int64_t>((int64_t(max_smem_bytes) - fixed) / (pitch + 8) / 2, 8);
    for (;;) {
        const bool piped = reduce_stages >= 2 && chunk >= 128;
        const int64_t pipe = piped ? int64_t(reduce_stages) * parts * chunk + 16 * reduce_stages : 0;
        const int64_t slots = (int64_t(max_smem_bytes) - fixed - pipe) / (pitch + 8);
        // three stages per transfer warp when there is room for at least four such warps, else two
        const int stages = slots >= 12 ? 3 : 2;
        const int64_t warps = std::min<int64_t>(slots / stages, 8);
        if (piped && reduce_chunk_bytes <= 0 && warps >= 1 && warps < std::min<int64_t>(2, alone) && chunk >= 2048) {
            chunk = chunk / 2 / 128 * 128;
            continue;
        }
        if (warps < 1 && piped) {
            // a long row leaves no room for the transfer rings: halve the chunk, and without any room left fall back
            // to the register path
            chunk = chunk > 128 ? std::max<int64_t>(128, chunk / 2 / 128 * 128) : 0;
            continue;
        }
        c.ring.stages = stages;
        c.ring.warps = warps < 1 ? 0 : int(warps);
        c.reduce_stages = piped ? reduce_stages : 0;
        c.reduce_chunk_bytes = piped ? int(chunk) : 0;
        c.ring.smem_bytes = size_t(c.ring.warps) * stages * (pitch + 8) + size_t(fixed - 256) + size_t(pipe);
        return c;
    }
}

cudaError_t launch_stage(const StageParams* params, LaunchShape shape, size_t smem, cudaStream_t stream) {
    return launch_pair<StageParams>(stage_kernel, stage_multi_kernel, params, shape, kStageThreads, smem, stream);
}
cudaError_t launch_plan(const PlanParams* params, LaunchShape shape, size_t smem, cudaStream_t stream) {
    return launch_pair<PlanParams>(plan_kernel, plan_multi_kernel, params, shape, kPlanThreads, smem, stream);
}
cudaError_t launch_pull(const PullParams* params, LaunchShape shape, int warps, size_t smem, cudaStream_t stream) {
    return launch_pair<PullParams>(pull_kernel, pull_multi_kernel, params, shape, warps * 32, smem, stream);
}
cudaError_t launch_reduce(const ReduceParams* params, LaunchShape shape, cudaStream_t stream) {
    return launch_pair<ReduceParams>(reduce_kernel, reduce_multi_kernel, params, shape, kReduceThreads, 0, stream);
}
cudaError_t launch_barrier(const BarrierParams* params, LaunchShape shape, cudaStream_t stream) {
    return launch_pair<BarrierParams>(barrier_kernel, barrier_multi_kernel, params, shape, 32, 0, stream);
}

namespace {
// Cooperative launch of a two-parameter-block kernel: fails instead of deadlocking if the grid cannot be resident at once.
cudaError_t launch_cooperative(const void* single, const void* multi_fn, const void* first, const void* second, LaunchShape shape, int warps,
                               size_t smem, cudaStream_t stream, size_t (*granted)[64]) {
    const bool multi = shape.ranks_y > 1;
    const void* fn = multi ? multi_fn : single;
    if (smem > 48 * 1024) {
        // as in launch_pair: raise the limit once per (kernel, device), and only when it grows
        int device = 0;
        cudaGetDevice(&device);
        size_t& have = granted[multi ? 1 : 0][device & 63];
        if (smem > have) {
            cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
            if (e != cudaSuccess) return e;
            have = smem;
        }
    }
    const dim3 grid(shape.grid_x, multi ? shape.ranks_y : 1);
    // multi: the kernel takes the two device arrays; single: the two blocks by value
    void* args_multi[2] = {(void*)&first, (void*)&second};
    void* args_single[2] = {(void*)first, (void*)second};
    return cudaLaunchCooperativeKernel(fn, grid, dim3(warps * 32), multi ? args_multi : args_single, smem, stream);
}
}  // namespace

cudaError_t launch_fused_cached_dispatch(const StageParams* stage, const PullParams* pull, LaunchShape shape, int warps, size_t smem,
                                         cudaStream_t stream) {
    static thread_local size_t granted[2][64] = {};
    return launch_cooperative((const void*)fused_cached_dispatch_kernel, (const void*)fused_cached_dispatch_multi_kernel, stage, pull, shape,
                              warps, smem, stream, granted);
}

cudaError_t launch_fused_fresh_dispatch(const StageParams* stage, const PlanParams* plan, const PullParams* pull, LaunchShape shape, int warps,
                                        size_t smem, cudaStream_t stream) {
    const bool multi = shape.ranks_y > 1;
    const void* fn = multi ? (const void*)fused_fresh_dispatch_multi_kernel : (const void*)fused_fresh_dispatch_kernel;
    static thread_local size_t granted[2][64] = {};
    if (smem > 48 * 1024) {
        int device = 0;
        cudaGetDevice(&device);
        size_t& have = granted[multi ? 1 : 0][device & 63];
        if (smem > have) {
            cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
            if (e != cudaSuccess) return e;
            have = smem;
        }
    }
    const dim3 grid(shape.grid_x, multi ? shape.ranks_y : 1);
    void* args_multi[3] = {(void*)&stage, (void*)&plan, (void*)&pull};
    void* args_single[3] = {(void*)stage, (void*)plan, (void*)pull};
    return cudaLaunchCooperativeKernel(fn, grid, dim3(warps * 32), multi ? args_multi : args_single, smem, stream);
}

cudaError_t launch_combine(const CombineParams* params, LaunchShape shape, size_t smem, cudaStream_t stream, bool cooperative) {
    if (!cooperative) return launch_pair<CombineParams>(combine_kernel, combine_multi_kernel, params, shape, kCombineThreads, smem, stream);
    const bool multi = shape.ranks_y > 1;
    const void* fn = multi ? (const void*)combine_multi_kernel : (const void*)combine_kernel;
    static thread_local size_t granted[2][64] = {};
    if (smem > 48 * 1024) {
        int device = 0;
        cudaGetDevice(&device);
        size_t& have = granted[multi ? 1 : 0][device & 63];
        if (smem > have) {
            cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
            if (e != cudaSuccess) return e;
            have = smem;
        }
    }
    const dim3 grid(shape.grid_x, multi ? shape.ranks_y : 1);
    void* args[1] = {multi ? (void*)&params : (void*)params};
    return cudaLaunchCooperativeKernel(fn, grid, dim3(kCombineThreads), args, smem, stream);
}

cudaError_t launch_gate(int* gate, uint64_t timeout_ns, cudaStream_t stream) {
    gate_kernel<<<1, 1, 0, stream>>>(gate, timeout_ns);
    return cudaGetLastError();
}

cudaError_t launch_local_combine(const LocalCombineParams* params, LaunchShape shape, cudaStream_t stream) {
    return launch_pair<LocalCombineParams>(local_combine_kernel, local_combine_multi_kernel, params, shape, kReduceThreads, 0, stream);
}

int kernel_table(KernelInfo* out, int capacity) {
    struct Entry {
        const char* name;
        const void* fn;
    };
    const Entry entries[] = {
        {"stage", (const void*)stage_kernel},   {"plan", (const void*)plan_kernel},     {"pull", (const void*)pull_kernel},
        {"combine", (const void*)combine_kernel}, {"reduce", (const void*)reduce_kernel}, {"barrier", (const void*)barrier_kernel},
        {"local_combine", (const void*)local_combine_kernel}, {"fused_cached_dispatch", (const void*)fused_cached_dispatch_kernel},
        {"fused_fresh_dispatch", (const void*)fused_fresh_dispatch_kernel},
    };
    int n = 0;
    for (const Entry& e : entries) {
        if (n >= capacity) break;
        cudaFuncAttributes a{};
        if (cudaFuncGetAttributes(&a, e.fn) != cudaSuccess) {
            cudaGetLastError();
            continue;
        }
        out[n++] = KernelInfo{e.name, a.numRegs, int(a.sharedSizeBytes), a.maxThreadsPerBlock, int(a.constSizeBytes)};
    }
    return n;
}

}  // namespace nep
