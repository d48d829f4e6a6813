/**
 * @file config.hpp
 * Compile-time feature macros and the defaults of the run-time tuning table.
 *
 * The reference generates two headers from CMake cache variables
 * (cmake/Al_config.hpp.in:9-131, cmake/tuning_params.hpp.in:36-89).  Here the
 * feature macros stay compile-time (they change which code exists), while
 * every tuning value is only a *default*: al/tuning.hpp reads the matching
 * environment variable at Initialize() and exposes setters, so that a tuned
 * table for 2/4/8 GPUs can be applied without a rebuild.
 */
#pragma once

#define AL_VERSION_MAJOR 0
#define AL_VERSION_MINOR 1
#define AL_VERSION_PATCH 0
#define AL_VERSION "0.1.0"

// ---- feature macros (names follow cmake/Al_config.hpp.in so user code that
// tests them keeps compiling) ------------------------------------------------
#ifndef AL_NO_CUDA
#define AL_HAS_CUDA 1
#define AL_HAS_DEVICE 1          // the sm_100a peer-memory backend
#define AL_HAS_HOST_TRANSFER 1   // host-staged fallback backend
#define AL_HAS_RMA 1             // Al::ext put/notify/wait/sync
#define AL_HAS_HALF 1
#define AL_HAS_BFLOAT 1
#endif
#define AL_HAS_HOST 1            // shared-memory CPU backend (the MPI backend's role)

// Several user threads may call into the library concurrently (each on its
// own communicator).  The reference makes this a build option
// (CMakeLists.txt:60-159, AL_THREAD_MULTIPLE); the progress engine here always
// uses the multi-producer input queue, so the macro is always defined.
#define AL_THREAD_MULTIPLE 1

// ---- sizes that must be compile-time constants ------------------------------
#define AL_CACHE_LINE_SIZE 64
#define AL_DESTRUCTIVE_INTERFERENCE_SIZE 128

/** Largest communicator the device kernels are compiled for (one NVSwitch domain of B200s). */
#define AL_MAX_DEVICE_RANKS 8
/** Largest grid.x any collective kernel uses; sizes the per-CTA flag arrays. */
#define AL_MAX_CTAS 160

// ---- defaults of run-time tunables (see al/tuning.hpp) ----------------------
#define AL_PE_NUM_CONCURRENT_OPS_DEFAULT 4
#define AL_PE_NUM_STREAMS 64
#define AL_PE_NUM_PIPELINE_STAGES 2
#define AL_PE_INPUT_QUEUE_SIZE 8192
#define AL_SYNC_MEM_PREALLOC_DEFAULT 1024
#define AL_CUDA_STREAM_POOL_SIZE_DEFAULT 4
