// Out-of-band bootstrap without MPI.
//
// The library never exchanges ProcessInfo itself (the reference leaves that
// to MPI_Alltoall in the application, examples/allreduce.cpp:52-77).  This
// helper does the same three-call protocol through a rendezvous directory on
// the local file system: every rank writes one small file per peer and polls
// for the files addressed to it.  The launcher `ibcomm_run` creates the
// directory and sets
//
//   IBCOMM_RANK, IBCOMM_WORLD_SIZE, IBCOMM_BOOTSTRAP_DIR, IBCOMM_LOCAL_RANK
//
// (RANK / WORLD_SIZE / LOCAL_RANK as set by torchrun are accepted too).
#pragma once

#include <string>

#include "ibcomm/communicator.h"

namespace ibcomm {

struct BootstrapEnv {
  int rank = 0;
  int world_size = 1;
  int local_rank = 0;
  std::string dir;  // empty when world_size == 1 and nothing was set
};

BootstrapEnv ReadBootstrapEnv();

// CreateQueuePair for every peer, exchange, RegisterQueuePair, RegisterMyself.
// `tag` separates several communicators that share one directory.
void ConnectAll(Communicator* comm, const BootstrapEnv& env, const std::string& tag = "c0",
                int timeout_ms = 60000);

// Sum of one integer over all ranks, through rank 0 (tester exit status).
long long SumOverRanks(Communicator* comm, long long value);

}  // namespace ibcomm
