// The generic collective kernel: publish -> handshake -> pull/reduce, chunked
// through the double-buffered staging area.  One template serves all nine
// collectives; Ti/Tw/To are the user-input, wire (staging) and user-output
// element types and Red the reduction functor.  Pure data-movement collectives
// instantiate it once with byte elements.
#pragma once
#include "datamove.cuh"

namespace Al {
namespace internal {
namespace device {

template <typename Ti, typename Tw, typename To, typename Red>
__global__ void __launch_bounds__(512) coll_kernel(const __grid_constant__ CollParams P, Red red) {
  const Workspace& ws = P.ws;
  const int p = ws.p;
  const int rank = P.rank0 + (int)blockIdx.y;
  const unsigned cta = blockIdx.x, nct = gridDim.x;
  if (poisoned(ws, rank)) return;

  const DevColl kind = (DevColl)P.kind;
  const CountTable& T = P.tab[rank];
  const size_t half = ws.half_bytes;
  const size_t full_e = half / sizeof(Tw);
  const size_t cap_b = (half / (size_t)p) / 256 * 256;
  const size_t cap_e = cap_b / sizeof(Tw);
  constexpr size_t VEC = 16 / sizeof(Tw);  // split boundaries stay 16-byte aligned in staging
  const Ti* send = (const Ti*)P.send[rank];
  To* recv = (To*)P.recv[rank];
  const int root = P.root;

  __shared__ uint64_t s_chunks;
  uint64_t G = P.local_chunks[rank];

  for (uint64_t c = 0; c < G; ++c) {
    const int par = (int)((P.seq + c) & 1);
    char* mystage = ws.stage[rank] + (size_t)par * half;
    size_t lo, hi;

    // ------------------------------ publish --------------------------------
    switch (kind) {
      case DevColl::allreduce:
      case DevColl::reduce: {
        const size_t base = c * full_e, len = clamp_len(P.count, base, full_e);
        split_range(len, cta, nct, VEC, lo, hi);
        if (send && hi > lo) cta_convert<Ti, Tw>((Tw*)mystage + lo, send + base + lo, hi - lo);
        break;
      }
      case DevColl::bcast: {
        if (rank != root) break;
        const size_t base = c * full_e, len = clamp_len(P.count, base, full_e);
        split_range(len, cta, nct, VEC, lo, hi);
        if (send && hi > lo) cta_convert<Ti, Tw>((Tw*)mystage + lo, send + base + lo, hi - lo);
        break;
      }
      case DevColl::allgather:
      case DevColl::gather: {
        const size_t base = c * full_e, len = clamp_len(T.send_counts[rank], base, full_e);
        split_range(len, cta, nct, VEC, lo, hi);
        if (send && hi > lo) cta_convert<Ti, Tw>((Tw*)mystage + lo, send + base + lo, hi - lo);
        break;
      }
      case DevColl::reduce_scatter:
      case DevColl::alltoall:
      case DevColl::scatter: {
        if (kind == DevColl::scatter && rank != root) break;
        const size_t base = c * cap_e;
        for (int d = 0; d < p; ++d) {
          const size_t cnt = kind == DevColl::reduce_scatter ? T.recv_counts[d] : T.send_counts[d];
          const size_t len = clamp_len(cnt, base, cap_e);
          split_range(len, cta, nct, VEC, lo, hi);
          if (send && hi > lo)
            cta_convert<Ti, Tw>((Tw*)(mystage + (size_t)d * cap_b) + lo, send + T.send_displs[d] + base + lo, hi - lo);
        }
        break;
      }
      case DevColl::barrier: break;
    }

    // ------------------------------ handshake A ----------------------------
    const uint64_t e = make_epoch(P.seq, c + 1);
    arrive_and_post(ws, rank, FlagLayout::off_A, 0, e, c == 0, (int)(P.seq & 1), P.local_chunks[rank]);
    if (!wait_all(ws, rank, FlagLayout::off_A, 0, e, P.timeout_ns)) return;
    if (c == 0) {
      if (threadIdx.x == 0) {
        uint64_t g = 1;
        for (int r = 0; r < p; ++r) {
          const uint64_t m = ld_relaxed_sys(flag_slot(ws.flags[rank], FlagLayout::off_meta, (int)(P.seq & 1) * kMaxRanks + r));
          g = m > g ? m : g;
        }
        s_chunks = g;
      }
      __syncthreads();
      G = s_chunks;
    }

    // ------------------------------ consume --------------------------------
    char* stage_par[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) stage_par[r] = r < p ? ws.stage[r] + (size_t)par * half : nullptr;

    switch (kind) {
      case DevColl::allreduce: {
        const size_t base = c * full_e, len = clamp_len(P.count, base, full_e);
        if (!P.two_phase) {
          split_range(len, cta, nct, VEC, lo, hi);
          if (recv && hi > lo)
            cta_reduce<Tw, To, Red>(recv + base + lo, stage_par, lo * sizeof(Tw), p, hi - lo, red, P.scale, P.int_div);
          break;
        }
        // phase 1: reduce the slice this rank owns, in place in its own staging
        size_t s_lo, s_hi;
        split_range(len, (unsigned)rank, (unsigned)p, VEC, s_lo, s_hi);
        split_range(s_hi - s_lo, cta, nct, VEC, lo, hi);
        if (hi > lo)
          cta_reduce<Tw, Tw, Red>((Tw*)mystage + s_lo + lo, stage_par, (s_lo + lo) * sizeof(Tw), p, hi - lo, red,
                                  P.scale, P.int_div);
        arrive_and_post(ws, rank, FlagLayout::off_B, 1, e, false, 0, 0);
        if (!wait_all(ws, rank, FlagLayout::off_B, 1, e, P.timeout_ns)) return;
        // phase 2: collect every owner's slice
        for (int s = 0; s < p; ++s) {
          split_range(len, (unsigned)s, (unsigned)p, VEC, s_lo, s_hi);
          split_range(s_hi - s_lo, cta, nct, VEC, lo, hi);
          if (recv && hi > lo) {
            if constexpr (std::is_same<Tw, To>::value) {
              cta_copy((char*)(recv + base + s_lo + lo), stage_par[s] + (s_lo + lo) * sizeof(Tw), (hi - lo) * sizeof(Tw), true);
            } else {
              char* one[kMaxRanks] = {stage_par[s]};
              cta_reduce<Tw, To, RedNone>(recv + base + s_lo + lo, one, (s_lo + lo) * sizeof(Tw), 1, hi - lo, RedNone(), 1.0, 1);
            }
          }
        }
        break;
      }
      case DevColl::reduce: {
        if (rank != root) break;
        const size_t base = c * full_e, len = clamp_len(P.count, base, full_e);
        split_range(len, cta, nct, VEC, lo, hi);
        if (recv && hi > lo)
          cta_reduce<Tw, To, Red>(recv + base + lo, stage_par, lo * sizeof(Tw), p, hi - lo, red, P.scale, P.int_div);
        break;
      }
      case DevColl::reduce_scatter: {
        const size_t base = c * cap_e, len = clamp_len(T.recv_counts[rank], base, cap_e);
        split_range(len, cta, nct, VEC, lo, hi);
        if (recv && hi > lo)
          cta_reduce<Tw, To, Red>(recv + base + lo, stage_par, (size_t)rank * cap_b + lo * sizeof(Tw), p, hi - lo, red,
                                  P.scale, P.int_div);
        break;
      }
      case DevColl::allgather:
      case DevColl::gather: {
        if (kind == DevColl::gather && rank != root) break;
        const size_t base = c * full_e;
        for (int r = 0; r < p; ++r) {
          const size_t len = clamp_len(T.recv_counts[r], base, full_e);
          split_range(len, cta, nct, VEC, lo, hi);
          if (recv && hi > lo) {
            if constexpr (std::is_same<Tw, To>::value)
              cta_copy((char*)(recv + T.recv_displs[r] + base + lo), stage_par[r] + lo * sizeof(Tw), (hi - lo) * sizeof(Tw), true);
          }
        }
        break;
      }
      case DevColl::alltoall: {
        const size_t base = c * cap_e;
        for (int r = 0; r < p; ++r) {
          const size_t len = clamp_len(T.recv_counts[r], base, cap_e);
          split_range(len, cta, nct, VEC, lo, hi);
          if (recv && hi > lo) {
            if constexpr (std::is_same<Tw, To>::value)
              cta_copy((char*)(recv + T.recv_displs[r] + base + lo), stage_par[r] + (size_t)rank * cap_b + lo * sizeof(Tw),
                       (hi - lo) * sizeof(Tw), true);
          }
        }
        break;
      }
      case DevColl::bcast: {
        if (rank == root) break;
        const size_t base = c * full_e, len = clamp_len(P.count, base, full_e);
        split_range(len, cta, nct, VEC, lo, hi);
        if (recv && hi > lo) {
          if constexpr (std::is_same<Tw, To>::value)
            cta_copy((char*)(recv + base + lo), stage_par[root] + lo * sizeof(Tw), (hi - lo) * sizeof(Tw), true);
        }
        break;
      }
      case DevColl::scatter: {
        const size_t base = c * cap_e, len = clamp_len(T.recv_counts[rank], base, cap_e);
        split_range(len, cta, nct, VEC, lo, hi);
        if (recv && hi > lo) {
          if constexpr (std::is_same<Tw, To>::value)
            cta_copy((char*)(recv + base + lo), stage_par[root] + (size_t)rank * cap_b + lo * sizeof(Tw),
                     (hi - lo) * sizeof(Tw), true);
        }
        break;
      }
      case DevColl::barrier: break;
    }
  }

  if (G > 1) {
    // Both halves were used: make sure every peer is done reading before the
    // next launch (which may start on either half) overwrites them.
    const uint64_t e = make_epoch(P.seq, 1);
    arrive_and_post(ws, rank, FlagLayout::off_C, 2, e, false, 0, 0);
    (void)wait_all(ws, rank, FlagLayout::off_C, 2, e, P.timeout_ns);
  }
}

}  // namespace device
}  // namespace internal
}  // namespace Al
