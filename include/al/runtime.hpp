/**
 * @file runtime.hpp
 * Library life cycle and access to the process-wide singletons.
 *
 * Parity: Al::Initialize / Finalize / Initialized (include/Al.hpp:73-104,
 * src/Al.cpp:118-194).  Initialize is idempotent; it discovers the rank from
 * the launcher environment (no MPI_Init), connects the control plane, creates
 * the progress engine (thread started on first use unless
 * AL_PE_START_ON_DEMAND=0), initialises the CUDA layer when a device is
 * usable, and installs the fatal-signal handler unless
 * AL_DISABLE_SIGNAL_HANDLER is set.  Finalize tears down in reverse order and
 * writes the trace file when tracing is on.
 */
#pragma once
#include <vector>

#include "al/bootstrap.hpp"
#include "al/progress.hpp"

namespace Al {

void Initialize(int& argc, char**& argv);
void Initialize();
void Finalize();
bool Initialized();
/**
 * World ranks whose processes still hold their control connection, this one
 * included.  After a rank was lost the survivors build a communicator over
 * exactly these (HostCommunicator::from_ranks, DeviceCommunicator::from_ranks)
 * and carry on; the reference has no counterpart (its communicators are fixed
 * at creation and a lost rank ends the job).
 */
std::vector<int> AliveRanks();

namespace internal {
/** The control-plane world; throws unless the library is initialised. */
World* get_world();
/** True when a CUDA device is usable in this process (false on hosts without a driver). */
bool cuda_available();
}  // namespace internal
}  // namespace Al
