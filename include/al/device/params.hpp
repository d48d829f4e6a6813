/**
 * @file params.hpp
 * Plain-data structures shared between the host runtime and the device
 * kernels: the per-communicator workspace description, the arguments of one
 * collective launch and the status record a kernel fills when a wait runs out.
 *
 * Device protocol in one paragraph.  Every rank owns, in peer-mapped
 * ("symmetric") memory, a staging area of two halves and a flag area.  A
 * collective with sequence number k proceeds in chunks; in chunk c every rank
 * (1) copies ("publishes") its contribution into staging half (k+c)&1 with
 * all of its CTAs; the CTA that finishes last (2) stores the epoch
 * (k<<24 | c+1) into slot A[me] of every rank's flag area with release
 * semantics at system scope; every CTA then (3) waits, with a time budget,
 * until slots A[r] of its own flag area reached that epoch for every r, and
 * (4) pulls or reduces what it needs from the peers' staging halves with
 * ordinary 16-byte loads over NVLink.  Two-phase algorithms repeat the
 * handshake on the B flags.  Every chunk makes every rank wait for every
 * rank, so two halves suffice; a multi-chunk launch ends with a C-flag
 * barrier so that the next launch may start on either half.  Epochs only
 * grow, so flags are never reset.
 */
#pragma once
#include <cstddef>
#include <cstdint>

#include "al/config.hpp"

namespace Al {
namespace internal {
namespace device {

constexpr int kMaxRanks = AL_MAX_DEVICE_RANKS;
constexpr int kMaxCtas = AL_MAX_CTAS;

/**
 * Layout of one rank's flag area in units of uint64_t.  Every remotely
 * written word sits in its own 32-byte sector (stride 4 words).
 */
struct FlagLayout {
  static constexpr size_t stride = 4;
  static constexpr size_t off_A = 0;                                       // [kMaxRanks]
  static constexpr size_t off_B = off_A + kMaxRanks * stride;              // [kMaxRanks]
  static constexpr size_t off_C = off_B + kMaxRanks * stride;              // [kMaxRanks]
  static constexpr size_t off_meta = off_C + kMaxRanks * stride;           // [2][kMaxRanks]
  static constexpr size_t off_p2p_sent = off_meta + 2 * kMaxRanks * stride;   // [kMaxRanks], written by the sender
  static constexpr size_t off_p2p_acked = off_p2p_sent + kMaxRanks * stride;  // [kMaxRanks], written by the receiver
  static constexpr size_t off_rma = off_p2p_acked + kMaxRanks * stride;       // [kMaxRanks] notify counters
  static constexpr size_t off_halo = off_rma + kMaxRanks * stride;         // [4] ready-from-lo, ready-from-hi, data-from-lo, data-from-hi
  // Words below are only touched by the owning GPU.
  static constexpr size_t off_arrive = off_halo + 4 * stride;              // [2][4] CTA arrival counters (A, B, C, spare) per round parity
  static constexpr size_t off_status = off_arrive + 8 * stride;            // device-local copy of the status code
  static constexpr size_t off_p2p_arrive = off_status + stride;            // [2][16] per-item CTA arrival counters per piece parity
  static constexpr size_t off_p2p_ready = off_p2p_arrive + 32 * stride;    // [kMaxRanks], written by the receiver into the SENDER's area:
                                                                            //   word 0 = number of the message's first piece + 1, word 1 = descriptor of its buffer
  static constexpr size_t off_p2p_posted = off_p2p_ready + kMaxRanks * stride;  // [16] plain words, local: last piece each item of the running launch posted
  static constexpr size_t off_ring_arrive = off_p2p_posted + 16;           // [3][kRingDepth] plain words, local: CTA arrival counters of the
                                                                            //   ring-pipelined kernels, per CTA group and ring slot
  static constexpr size_t words = off_ring_arrive + 3 * 8;
  static constexpr size_t bytes = (words * 8 + 4095) / 4096 * 4096;
};

/** Most chunks a ring-pipelined kernel keeps in flight in the staging area (FlagLayout::off_ring_arrive). */
constexpr int kRingDepth = 8;
static_assert(FlagLayout::bytes == 4096, "the flag area is one page (the allocation-free entry point's scratch layout depends on it)");

/** Why a kernel gave up. */
enum StatusCode : uint32_t {
  kStatusOk = 0,
  kStatusTimeout = 1,      ///< a flag wait exceeded its time budget
  kStatusPoisoned = 2,     ///< an earlier kernel of this communicator had failed; this one did nothing
  kStatusMismatch = 3      ///< the ranks entered one operation with different protocols (e.g. one rank passed a
                           ///< registered / symmetric buffer and another a private one); `seen` = the other tag
};

/**
 * Protocol tag every kernel publishes when it enters an operation, so that ranks which chose
 * different kernels for the same operation find out at once instead of waiting for flags that
 * never come.  The choice depends on rank-local facts (is this rank's buffer registered?), which
 * is why it has to be compared.
 */
enum ProtoTag : uint64_t {
  kProtoNone = 0,
  kProtoStaged = 1,        ///< generic kernel through the staging halves (any algorithm of it)
  kProtoNvlsStaged = 2,    ///< NVLS allreduce through the multicast-bound staging
  kProtoNvlsZeroCopy = 3,  ///< NVLS allreduce on symmetric user buffers
  kProtoWindow = 4         ///< reduce_scatter / allgather / alltoall / bcast straight on registered buffers
};

/**
 * The four meta words rank r publishes in slot [parity][r] of every rank's flag area:
 *   word 0  chunk count of the operation (with the first A flag)
 *   word 1  ProtoTag << 8 | DevColl kind (with "entered")
 *   word 2  descriptor of the receive buffer, word 3 of the send buffer (window kernels)
 */
constexpr int kMetaChunks = 0, kMetaProto = 1, kMetaRecvDesc = 2, kMetaSendDesc = 3;

/** Registered buffers ("windows"): every rank can address every rank's buffer of a window. */
constexpr int kMaxWindows = 32;
struct WindowTable {
  char* peer[kMaxWindows][kMaxRanks];    ///< address, in this process, of rank r's buffer of window w (nullptr: free slot)
  size_t bytes[kMaxWindows][kMaxRanks];  ///< its length
  char* mc[kMaxWindows];                 ///< NVLink-multicast alias of the window (same offset on every rank), or nullptr
};
/** Buffer descriptor: (window + 1) << 48 | byte offset inside this rank's buffer of the window; 0 = not registered. */
constexpr uint64_t make_desc(int window, size_t offset) { return ((uint64_t)(window + 1) << 48) | (uint64_t)offset; }
constexpr int desc_window(uint64_t d) { return (int)(d >> 48) - 1; }
constexpr size_t desc_offset(uint64_t d) { return (size_t)(d & ((uint64_t{1} << 48) - 1)); }

/** Written by a kernel into pinned host memory; read by the host in Wait/Test and before each launch. */
struct DeviceStatus {
  uint32_t code;    ///< StatusCode
  uint32_t rank;    ///< rank that gave up
  uint32_t peer;    ///< rank it was waiting for
  uint32_t where;   ///< 0: A flags, 1: B flags, 2: C flags, 3: p2p credit, 4: p2p data, 5: rma, 6: a bulk copy that did not complete, 7: protocol comparison
  uint64_t epoch;   ///< epoch it was waiting for
  uint64_t seen;    ///< value it last saw
};

/**
 * Low-latency packets (small allreduce / reduce_scatter / allgather / alltoall): every 8 bytes carry 4 bytes
 * of payload and the 4-byte epoch of the operation, written and read as 16-byte vectors whose two halves
 * are each delivered whole.  The receiver polls the data itself, so there is no flag round and no fence
 * between the data and a flag (the role of NCCL's LL protocol, which the reference gets from ncclAllReduce
 * & co. at these sizes).  One slot per (parity of the operation number, source rank).
 */
constexpr size_t kLLPayloadBytes = 1048576;
constexpr size_t kLLSlotBytes = 2 * kLLPayloadBytes;
constexpr size_t kLLAreaBytes = 2 * (size_t)kMaxRanks * kLLSlotBytes;
/**
 * Small point-to-point messages travel as the same kind of packets: a ring of packet slots per ordered pair
 * of ranks, [source][piece number % mbox_slots] of Workspace::p2p_ll_slot_bytes each (twice the largest
 * payload, fixed when the communicator is created), placed behind the collectives' packet area (at
 * ll[r] + kLLAreaBytes).  The packets' epoch is the pair's piece number + 1.
 */
constexpr size_t kP2PLLMaxPayloadBytes = size_t{8} << 20;  ///< upper bound of the tunable payload limit

/** Workspace of one communicator as seen from the launching process. */
struct Workspace {
  char* stage[kMaxRanks];        ///< staging base (two halves, contiguous) of every rank
  uint64_t* flags[kMaxRanks];    ///< flag area of every rank
  char* mbox[kMaxRanks];         ///< p2p mailbox area of every rank: [src][2 slots]
  char* ll[kMaxRanks];           ///< low-latency packet area of every rank: [parity][src][kLLSlotBytes], then the
                                 ///< point-to-point packet slots [src][mbox_slots][p2p_ll_slot_bytes]
  char* mc_stage;                ///< NVLink-multicast alias of the staging area, or nullptr
  DeviceStatus* status;          ///< pinned host record (device-visible address)
  uint64_t* stamps;              ///< nullptr, or 4 words of this GPU's memory that the small-message kernels fill with
                                 ///< %globaltimer at entry / data sent / data seen / exit (latency breakdowns)
  size_t half_bytes;             ///< size of one staging half
  size_t mbox_slot_bytes;        ///< size of one mailbox slot
  size_t p2p_ll_slot_bytes;      ///< size of one point-to-point packet slot (0: no packet slots)
  int mbox_slots;                ///< slots per (source, destination) ring
  int p;                         ///< communicator size
};

/** Operation selector of the collective kernels. */
enum class DevColl : int {
  allreduce = 0, reduce, reduce_scatter, allgather, alltoall, bcast, gather, scatter, barrier
};

/** Per-rank element counts and displacements (vector collectives; uniform ones are synthesised). */
struct CountTable {
  size_t send_counts[kMaxRanks];
  size_t send_displs[kMaxRanks];
  size_t recv_counts[kMaxRanks];
  size_t recv_displs[kMaxRanks];
};

/**
 * Arguments of one launch.  A launch normally executes one rank (grid.y == 1).
 * When several ranks of a communicator live in one process on one device
 * (single-GPU emulation used by tests), one cooperative launch executes all
 * of them: grid.y == number of local ranks and block (x, y) works for rank
 * rank0 + y.
 */
struct CollParams {
  Workspace ws;
  const void* send[kMaxRanks];   ///< indexed by rank; nullptr = contributes nothing
  void* recv[kMaxRanks];         ///< indexed by rank; nullptr = receives nothing
  CountTable tab[kMaxRanks];     ///< indexed by rank (only local ranks are filled)
  uint64_t local_chunks[kMaxRanks];
  uint64_t seq;
  uint64_t timeout_ns;
  size_t count;                  ///< uniform count (allreduce / reduce / bcast)
  double scale;                  ///< multiplies the result of a reduction (1/p for avg); 1 = none
  int int_div;                   ///< integer types: divide the result by this (avg); 1 = none
  int kind;                      ///< DevColl
  int op;                        ///< ReductionOperator
  int root;
  int rank0;
  int two_phase;                 ///< allreduce: 1 = reduce-scatter + allgather, 0 = every rank reduces everything
  int pipelined;                 ///< 1: half of the CTAs publish while the other half consumes (large uniform ops)
  size_t slot_elems;             ///< elements moved per slot and chunk (0 = the slot's capacity)
  int n_pub;                     ///< bulk-copy pipeline: number of publishing CTAs (0 = half of the grid)
  int own_direct;                ///< one-shot allreduce: a rank reads its own contribution from its send buffer instead of
                                 ///< pushing it into its own slot (same in / wire type, 16-byte aligned send buffer)
};

/**
 * Arguments of one launch of the window kernel: uniform reduce_scatter / allgather / alltoall / bcast
 * whose remote side is a registered buffer.  Indexed by rank like CollParams (one entry outside emulation).
 */
struct WinParams {
  Workspace ws;
  const WindowTable* windows;    ///< device memory of the launching process
  const void* send[kMaxRanks];
  void* recv[kMaxRanks];
  uint64_t send_desc[kMaxRanks]; ///< 0 when the send buffer is private
  uint64_t recv_desc[kMaxRanks];
  size_t count;                  ///< elements per rank slice (bcast: the whole vector)
  uint64_t seq;
  uint64_t timeout_ns;
  double scale;
  int int_div;
  int kind;                      ///< DevColl: reduce_scatter, allgather, alltoall or bcast
  int op;
  int root;
  int rank0;
  int allow_multimem;            ///< bit 0: multimem for reduce_scatter / bcast, bit 1: for allgather; 0: plain peer loads / stores only
};

/** Arguments of one launch of the low-latency kernel (kernels/ll.cu).  Indexed by rank like CollParams. */
struct LLParams {
  Workspace ws;
  const void* send[kMaxRanks];
  void* recv[kMaxRanks];
  size_t count;                  ///< elements: the vector (allreduce) or one rank's slice (the others)
  uint64_t seq;
  uint64_t timeout_ns;
  double scale;
  int int_div;
  int kind;                      ///< DevColl: allreduce, reduce_scatter, allgather or alltoall
  int op;
  int rank0;
  int two_phase;                 ///< allreduce only: reduce-scatter the vector in packets, then allgather the reduced slices in
                                 ///< packets (second half of every slot); a slice then holds at most kLLPayloadBytes / 2
};

/**
 * Row exchange (kernels/rows.cu): an alltoall(v) whose slices are sets of equally long rows that need not be
 * contiguous.  Row k of what a rank sends to peer d is read at
 *     send + send_peer_off[d] + id * send_row_stride,   id = send_first[d] + k, or send_idx[send_first[d] + k]
 * and row k of what it receives from rank r is written at
 *     recv + recv_peer_off[r] + id * recv_row_stride,   id = recv_first[r] + k, or recv_idx[recv_first[r] + k]
 * (offsets and strides in bytes, index arrays in device memory).  The pack before and the unpack after an
 * alltoall - a transposition for sequence <-> head exchanges, a gather / scatter by token index for expert
 * dispatch / combine - thereby happen inside the kernel's publish and consume steps.
 */
struct RowTable {
  size_t send_rows[kMaxRanks], send_first[kMaxRanks], send_peer_off[kMaxRanks];
  size_t recv_rows[kMaxRanks], recv_first[kMaxRanks], recv_peer_off[kMaxRanks];
};
struct RowsParams {
  Workspace ws;
  const void* send[kMaxRanks];
  void* recv[kMaxRanks];
  const long long* send_idx[kMaxRanks];  ///< nullptr: rows are taken in order
  const long long* recv_idx[kMaxRanks];
  RowTable tab[kMaxRanks];               ///< indexed by rank (local ranks only)
  uint64_t local_chunks[kMaxRanks];
  size_t row_bytes;
  size_t send_row_stride;
  size_t recv_row_stride;
  uint64_t seq;
  uint64_t timeout_ns;
  int rank0;
};

/** Arguments of one point-to-point launch (any mix of sends and receives). */
struct P2PParams {
  static constexpr int kMaxItems = 16;
  Workspace ws;
  const void* sbuf[kMaxItems];
  void* rbuf[kMaxItems];
  size_t bytes[kMaxItems];
  int peer[kMaxItems];
  int is_send[kMaxItems];
  int owner[kMaxItems];          ///< rank executing this item (emulation: several ranks per launch)
  uint64_t base[kMaxItems];      ///< pieces already moved between this pair in this direction (host-tracked)
  uint64_t rdesc[kMaxItems];     ///< receives: descriptor of the receive buffer when it is registered, else 0
  const WindowTable* windows;    ///< device memory of the launching process
  size_t rendezvous_bytes;       ///< messages of at least this size wait for the receiver and go straight into a registered buffer
  size_t ll_bytes;               ///< messages of at most this size (> 0) travel as packets (at most half a packet slot)
  uint64_t launch;               ///< number of this launch on the communicator (tags the local "posted" words)
  int ctas_per_item;
  int nitems;
  uint64_t timeout_ns;
};

}  // namespace device
}  // namespace internal
}  // namespace Al
