// The generic collective kernel: push -> handshake -> local consume, chunked
// through the double-buffered staging area.
//
// Every rank's staging half is divided into p slots of `cap_b` bytes, one per
// source rank.  In the publish step a rank reads its contribution once from the
// user's send buffer and STORES it into slot [me] of the destination rank's
// staging half over NVLink (remote stores are posted and do not stall the
// issuing threads the way remote loads do; measured on 8 GPUs, pulling with
// loads reached a third of the pushed bandwidth).  After the epoch handshake a
// rank finds everything it needs in its own memory and reduces / copies it to
// the user's receive buffer with local loads.  One template serves all nine
// collectives; Ti/Tw/To are the user-input, wire (staging) and user-output
// element types and Red the reduction functor.  Pure data-movement collectives
// instantiate it once with byte elements.  FAM says which operations an
// instantiation serves, so that the reducing instantiations (one per element
// type and operator) do not carry the code and registers of the data-movement
// operations and the byte instantiation none of the reductions.
#pragma once
#include "datamove.cuh"

namespace Al {
namespace internal {
namespace device {

constexpr int kFamAll = 0;     // every operation (mixed element types)
constexpr int kFamReduce = 1;  // allreduce, reduce, reduce_scatter (+ barrier)
constexpr int kFamMove = 2;    // allgather, alltoall, bcast, gather, scatter (+ barrier)

/** Whether an instantiation of family `fam` serves operation `kind`. */
inline bool family_serves(int fam, DevColl kind) {
  const bool reduces = kind == DevColl::allreduce || kind == DevColl::reduce || kind == DevColl::reduce_scatter;
  return fam == kFamAll || kind == DevColl::barrier || (fam == kFamReduce) == reduces;
}

template <typename Ti, typename Tw, typename To, typename Red, int FAM = kFamAll>
__global__ void __launch_bounds__(512) coll_kernel(const __grid_constant__ CollParams P, Red red) {
  constexpr bool kReduces = FAM != kFamMove, kMoves = FAM != kFamReduce;
  const Workspace& ws = P.ws;
  const int p = ws.p;
  const int rank = P.rank0 + (int)blockIdx.y;
  if (poisoned(ws, rank)) return;
  stamp(ws, 0);

  const DevColl kind = (DevColl)P.kind;
  const CountTable& T = P.tab[rank];
  // Operations that also exist as window kernels (registered buffers) announce which protocol this
  // rank runs, so that a rank that chose the other one is not left waiting (see protocols_agree).
  const uint64_t my_proto = proto_word(kProtoStaged, P.kind, P.two_phase | (P.pipelined << 1));
  const bool announces = kind == DevColl::reduce_scatter || kind == DevColl::allgather || kind == DevColl::alltoall ||
                         kind == DevColl::bcast;
  if (announces && blockIdx.x == 0) post_entered(ws, rank, P.seq, my_proto, 0, 0);
  const size_t half = ws.half_bytes;
  const size_t full_e = half / sizeof(Tw);
  const size_t cap_b = (half / (size_t)p) / 256 * 256;           // one slot per source rank
  const size_t cap_e = P.slot_elems ? P.slot_elems : cap_b / sizeof(Tw);  // elements moved per slot and chunk
  const size_t cap2_b = (half / 2 / (size_t)p) / 256 * 256;      // two-phase allreduce: two areas of p slots
  const size_t cap2_e = cap2_b / sizeof(Tw);
  const size_t area_b = half / 2 / 256 * 256;                    // byte offset of the second area
  constexpr size_t VEC = 16 / sizeof(Tw);  // split boundaries stay 16-byte aligned in staging
  const Ti* send = (const Ti*)P.send[rank];
  To* recv = (To*)P.recv[rank];
  const int root = P.root;
  // Small single-CTA messages: the CTA's threads split into p groups that serve all peers at once
  // instead of one peer after the other.
  const unsigned grp_lanes = blockDim.x / (unsigned)p;
  const unsigned grp = threadIdx.x / grp_lanes, lane = threadIdx.x % grp_lanes;
  constexpr size_t kSmallBytes = 65536;  // per-peer slice up to which the peers are served in parallel

  // ------------------------------ publish (remote stores) --------------------
  auto publish = [&](uint64_t c, unsigned part, unsigned nparts) {
    const int par = (int)((P.seq + c) & 1);
    char* all_stage[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) all_stage[r] = r < p ? ws.stage[r] + (size_t)par * half : nullptr;
    size_t lo, hi;
    switch (kind) {
      case DevColl::allreduce: if constexpr (kReduces) {
        if (!P.two_phase) {  // every rank gets every rank's whole chunk
          const size_t base = c * cap_e, len = clamp_len(P.count, base, cap_e);
          split_range(len, part, nparts, VEC, lo, hi);
          if (send && hi > lo) {
            if (P.own_direct) {  // the own contribution is read from the send buffer at reduce time: p-1 destinations
              char* others[kMaxRanks];
              int n = 0;
#pragma unroll
              for (int r = 0; r < kMaxRanks; ++r) {
                others[r] = nullptr;
                if (r < p && r != rank) others[n++] = all_stage[r];
              }
              cta_publish<Ti, Tw>(others, n, (size_t)rank * cap_b + lo * sizeof(Tw), send + base + lo, hi - lo);
            } else {
              cta_publish<Ti, Tw>(all_stage, p, (size_t)rank * cap_b + lo * sizeof(Tw), send + base + lo, hi - lo);
            }
          }
        } else {             // rank d gets slice d of every rank's chunk
          const size_t unit = (size_t)p * cap2_e, base = c * unit, len = clamp_len(P.count, base, unit);
          for (int i = 0; i < p; ++i) {
            const int d = (rank + 1 + i) % p;  // rotated start: at every step the destinations form a permutation
            size_t s_lo, s_hi;
            split_range(len, (unsigned)d, (unsigned)p, VEC, s_lo, s_hi);
            split_range(s_hi - s_lo, part, nparts, VEC, lo, hi);
            if (send && hi > lo)
              cta_publish<Ti, Tw>(&all_stage[d], 1, (size_t)rank * cap2_b + lo * sizeof(Tw), send + base + s_lo + lo, hi - lo);
          }
        }
        break;
      } break;
      case DevColl::reduce: if constexpr (kReduces) {
        const size_t base = c * cap_e, len = clamp_len(P.count, base, cap_e);
        split_range(len, part, nparts, VEC, lo, hi);
        if (send && hi > lo)
          cta_publish<Ti, Tw>(&all_stage[root], 1, (size_t)rank * cap_b + lo * sizeof(Tw), send + base + lo, hi - lo);
        break;
      } break;
      case DevColl::bcast: if constexpr (kMoves) {
        if (rank != root) break;
        const size_t base = c * full_e, len = clamp_len(P.count, base, full_e);
        split_range(len, part, nparts, VEC, lo, hi);
        if (send && hi > lo) cta_publish<Ti, Tw>(all_stage, p, lo * sizeof(Tw), send + base + lo, hi - lo);
        break;
      } break;
      case DevColl::allgather:
      case DevColl::gather: if constexpr (kMoves) {
        const size_t base = c * cap_e, len = clamp_len(T.send_counts[rank], base, cap_e);
        split_range(len, part, nparts, VEC, lo, hi);
        if (send && hi > lo) {
          if (kind == DevColl::allgather)
            cta_publish<Ti, Tw>(all_stage, p, (size_t)rank * cap_b + lo * sizeof(Tw), send + base + lo, hi - lo);
          else
            cta_publish<Ti, Tw>(&all_stage[root], 1, (size_t)rank * cap_b + lo * sizeof(Tw), send + base + lo, hi - lo);
        }
        break;
      } break;
      case DevColl::reduce_scatter:
      case DevColl::alltoall:
      case DevColl::scatter: {
        if constexpr (!kMoves) { if (kind != DevColl::reduce_scatter) break; }
        if constexpr (!kReduces) { if (kind == DevColl::reduce_scatter) break; }
        if (kind == DevColl::scatter && rank != root) break;
        const bool sc = kind == DevColl::scatter;
        const size_t unit = sc ? full_e : cap_e, base = c * unit;
        const size_t slot_off = sc ? 0 : (size_t)rank * cap_b;
        size_t maxlen = 0;
        for (int d = 0; d < p; ++d) {
          const size_t cnt = kind == DevColl::reduce_scatter ? T.recv_counts[d] : T.send_counts[d];
          const size_t len = clamp_len(cnt, base, unit);
          maxlen = len > maxlen ? len : maxlen;
        }
        if (grp_lanes >= 32 && maxlen * sizeof(Tw) <= kSmallBytes) {
          if ((int)grp < p && send) {
            const int d = (int)grp;
            const size_t cnt = kind == DevColl::reduce_scatter ? T.recv_counts[d] : T.send_counts[d];
            const size_t len = clamp_len(cnt, base, unit);
            split_range(len, part, nparts, VEC, lo, hi);
            if (hi > lo)
              group_publish<Ti, Tw>(all_stage[d] + slot_off + lo * sizeof(Tw), send + T.send_displs[d] + base + lo, hi - lo, lane, grp_lanes);
          }
          break;
        }
        // Every rank starts with a different destination (rank+1, rank+2, ...): at any moment the
        // ranks write to distinct peers instead of all converging on one GPU's ingress link.
        for (int i = 0; i < p; ++i) {
          const int d = (rank + 1 + i) % p;
          const size_t cnt = kind == DevColl::reduce_scatter ? T.recv_counts[d] : T.send_counts[d];
          const size_t len = clamp_len(cnt, base, unit);
          split_range(len, part, nparts, VEC, lo, hi);
          if (send && hi > lo)
            cta_publish<Ti, Tw>(&all_stage[d], 1, slot_off + lo * sizeof(Tw), send + T.send_displs[d] + base + lo, hi - lo);
        }
        break;
      }
      case DevColl::barrier: break;
    }
  };

  // ------------------------------ consume (local loads), single-phase kinds ---
  auto consume = [&](uint64_t c, unsigned part, unsigned nparts) {
    const int par = (int)((P.seq + c) & 1);
    char* mystage = ws.stage[rank] + (size_t)par * half;
    char* slot[kMaxRanks];    // my slots, one per source rank
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) slot[r] = mystage + (size_t)r * cap_b;
    size_t lo, hi;
    switch (kind) {
      case DevColl::allreduce:
      case DevColl::reduce: if constexpr (kReduces) {
        if (kind == DevColl::reduce && rank != root) break;
        const size_t base = c * cap_e, len = clamp_len(P.count, base, cap_e);
        split_range(len, part, nparts, VEC, lo, hi);
        if constexpr (std::is_same<Ti, Tw>::value) {
          if (P.own_direct && kind == DevColl::allreduce) slot[rank] = (char*)(send + base);
        }
        if (recv && hi > lo) {
          To* out = recv + base + lo;
          cta_reduce<Tw, To, Red>(&out, 1, slot, lo * sizeof(Tw), p, hi - lo, red, P.scale, P.int_div);
        }
        break;
      } break;
      case DevColl::reduce_scatter: if constexpr (kReduces) {
        const size_t base = c * cap_e, len = clamp_len(T.recv_counts[rank], base, cap_e);
        split_range(len, part, nparts, VEC, lo, hi);
        if (recv && hi > lo) {
          To* out = recv + base + lo;
          cta_reduce<Tw, To, Red>(&out, 1, slot, lo * sizeof(Tw), p, hi - lo, red, P.scale, P.int_div);
        }
        break;
      } break;
      case DevColl::allgather:
      case DevColl::gather:
      case DevColl::alltoall: if constexpr (kMoves) {
        if (kind == DevColl::gather && rank != root) break;
        const size_t base = c * cap_e;
        if constexpr (std::is_same<Tw, To>::value) {
          size_t maxlen = 0;
          for (int r = 0; r < p; ++r) {
            const size_t len = clamp_len(T.recv_counts[r], base, cap_e);
            maxlen = len > maxlen ? len : maxlen;
          }
          if (grp_lanes >= 32 && maxlen * sizeof(Tw) <= kSmallBytes) {
            if ((int)grp < p && recv) {
              const int r = (int)grp;
              const size_t len = clamp_len(T.recv_counts[r], base, cap_e);
              split_range(len, part, nparts, VEC, lo, hi);
              if (hi > lo)
                group_copy((char*)(recv + T.recv_displs[r] + base + lo), slot[r] + lo * sizeof(Tw), (hi - lo) * sizeof(Tw), true, lane, grp_lanes);
            }
            break;
          }
          for (int r = 0; r < p; ++r) {
            const size_t len = clamp_len(T.recv_counts[r], base, cap_e);
            split_range(len, part, nparts, VEC, lo, hi);
            if (recv && hi > lo)
              cta_copy((char*)(recv + T.recv_displs[r] + base + lo), slot[r] + lo * sizeof(Tw), (hi - lo) * sizeof(Tw), true);
          }
        }
        break;
      } break;
      case DevColl::bcast:
      case DevColl::scatter: if constexpr (kMoves) {
        if (kind == DevColl::bcast && rank == root) break;
        const size_t cnt = kind == DevColl::bcast ? P.count : T.recv_counts[rank];
        const size_t base = c * full_e, len = clamp_len(cnt, base, full_e);
        split_range(len, part, nparts, VEC, lo, hi);
        if (recv && hi > lo) {
          if constexpr (std::is_same<Tw, To>::value)
            cta_copy((char*)(recv + base + lo), mystage + lo * sizeof(Tw), (hi - lo) * sizeof(Tw), true);
        }
        break;
      } break;
      case DevColl::barrier: break;
    }
  };

  // =========================== pipelined schedule =============================
  // Large uniform reduce_scatter / allgather / alltoall: the lower half of the grid
  // only publishes (NVLink stores), the upper half only consumes (HBM traffic), so
  // chunk c+1 crosses the links while chunk c is copied out.  A slot is reused
  // every second chunk; the publisher waits for the consumers' C flag of the chunk
  // that used it before.
  if (P.pipelined && gridDim.x >= 2) {
    const unsigned n_pub = gridDim.x / 2, n_con = gridDim.x - n_pub;
    const uint64_t G = P.local_chunks[rank];
    if (blockIdx.x < n_pub) {
      for (uint64_t c = 0; c < G; ++c) {
        if (c >= 2 && !wait_all(ws, rank, FlagLayout::off_C, 2, make_epoch(P.seq, c - 1), P.timeout_ns)) return;
        publish(c, blockIdx.x, n_pub);
        arrive_and_post(ws, rank, FlagLayout::off_A, 0, n_pub, make_epoch(P.seq, c + 1), c == 0, (int)(P.seq & 1), G, my_proto);
      }
    } else {
      for (uint64_t c = 0; c < G; ++c) {
        if (!wait_all(ws, rank, FlagLayout::off_A, 0, make_epoch(P.seq, c + 1), P.timeout_ns)) return;
        if (c == 0 && !protocols_agree(ws, rank, P.seq, my_proto)) return;
        consume(c, blockIdx.x - n_pub, n_con);
        arrive_and_post(ws, rank, FlagLayout::off_C, 2, n_con, make_epoch(P.seq, c + 1), false, 0, 0);
      }
    }
    // Closing barrier: every peer has consumed every chunk, both halves are free.
    (void)wait_all(ws, rank, FlagLayout::off_C, 2, make_epoch(P.seq, G), P.timeout_ns);
    return;
  }

  // =========================== serial schedule ================================
  const unsigned cta = blockIdx.x, nct = gridDim.x;
  __shared__ uint64_t s_chunks;
  uint64_t G = P.local_chunks[rank];
  for (uint64_t c = 0; c < G; ++c) {
    publish(c, cta, nct);
    const uint64_t e = make_epoch(P.seq, c + 1);
    arrive_and_post(ws, rank, FlagLayout::off_A, 0, nct, e, c == 0, (int)(P.seq & 1), P.local_chunks[rank], my_proto);
    if (c == 0) stamp(ws, 1);
    if (!wait_all(ws, rank, FlagLayout::off_A, 0, e, P.timeout_ns)) return;
    if (c == 0) {
      stamp(ws, 2);
      if (p > 1 && !protocols_agree(ws, rank, P.seq, my_proto)) return;
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
    if (!kReduces || !(kind == DevColl::allreduce && P.two_phase)) {
      consume(c, cta, nct);
      continue;
    }
    if constexpr (kReduces) {
    // ---- two-phase allreduce ---------------------------------------------------
    const int par = (int)((P.seq + c) & 1);
    char* mystage = ws.stage[rank] + (size_t)par * half;
    const size_t unit = (size_t)p * cap2_e, base = c * unit, len = clamp_len(P.count, base, unit);
    // phase 1: reduce the slice this rank owns and push the result to everyone's second area
    char* slot2[kMaxRanks];
    Tw* outs[kMaxRanks];
    size_t lo, hi, s_lo, s_hi;
    split_range(len, (unsigned)rank, (unsigned)p, VEC, s_lo, s_hi);
    split_range(s_hi - s_lo, cta, nct, VEC, lo, hi);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      slot2[r] = mystage + (size_t)r * cap2_b;
      outs[r] = r < p ? (Tw*)(ws.stage[r] + (size_t)par * half + area_b + (size_t)rank * cap2_b) + lo : nullptr;
    }
    if (hi > lo) cta_reduce<Tw, Tw, Red>(outs, p, slot2, lo * sizeof(Tw), p, hi - lo, red, P.scale, P.int_div);
    arrive_and_post(ws, rank, FlagLayout::off_B, 1, nct, e, false, 0, 0);
    if (!wait_all(ws, rank, FlagLayout::off_B, 1, e, P.timeout_ns)) return;
    // phase 2: every owner's reduced slice is now in my second area
    for (int s = 0; s < p; ++s) {
      split_range(len, (unsigned)s, (unsigned)p, VEC, s_lo, s_hi);
      split_range(s_hi - s_lo, cta, nct, VEC, lo, hi);
      if (recv && hi > lo) {
        char* src = mystage + area_b + (size_t)s * cap2_b;
        if constexpr (std::is_same<Tw, To>::value) {
          cta_copy((char*)(recv + base + s_lo + lo), src + lo * sizeof(Tw), (hi - lo) * sizeof(Tw), true);
        } else {
          To* out = recv + base + s_lo + lo;
          cta_reduce<Tw, To, RedNone>(&out, 1, &src, lo * sizeof(Tw), 1, hi - lo, RedNone(), 1.0, 1);
        }
      }
    }
    }  // kReduces
  }

  stamp(ws, 3);
  if (G > 1) {
    // Both halves were used: make sure every peer is done with them before the
    // next launch (which may start on either half) writes into them.
    const uint64_t e = make_epoch(P.seq, 1);
    arrive_and_post(ws, rank, FlagLayout::off_C, 2, nct, e, false, 0, 0);
    (void)wait_all(ws, rank, FlagLayout::off_C, 2, e, P.timeout_ns);
  }
}

}  // namespace device
}  // namespace internal
}  // namespace Al
