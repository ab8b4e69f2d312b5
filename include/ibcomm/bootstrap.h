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
#include <vector>

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

// Environment of a communicator over a subset of the job's ranks: a member's
// rank is its position in `ranks`, the world size is the size of the list, and
// `*tag` gets a suffix naming the subset so that the rendezvous files do not
// collide with those of other communicators.  Every member calls with the
// same list.  This is how the survivors of a failed rank form a smaller world
// (the old communicator's collectives have returned TRANSPORT_ERROR by then).
// INVALID_ARGUMENT when this rank is not in the list or the list is malformed.
BootstrapEnv SubsetEnv(const BootstrapEnv& env, const std::vector<int>& ranks, std::string* tag);

// Sum of one integer over all ranks, through rank 0 (tester exit status).
long long SumOverRanks(Communicator* comm, long long value);

}  // namespace ibcomm
