// Internal layout of the data-parallel handle shared by dp.cu (communicator, peer mappings) and optim.cu (the sharded
// update kernel).
#pragma once
#include "common.cuh"

struct B2kDp {
  int rank = 0, world = 1, device = 0;
  void* comm = nullptr;                 // ncclComm_t
  uint32_t* barrier_word = nullptr;     // device word the barrier all-reduces
  unsigned char* handle_buf = nullptr;  // [world][64] device staging for the exchange of memory handles
  void* opened[256];                    // peer mappings to close in b2k_dp_destroy
  int n_opened = 0;
};
