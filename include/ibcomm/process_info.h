// Endpoint descriptor exchanged out-of-band by the application, one per
// (communicator, peer) pair, exactly like the reference's queue-pair triple
// (ibverbs_communicator.h:24-28).  It stays a 3-integer POD so it can travel
// through MPI_Alltoall, a torch.distributed store or a file.
//
//   lid   16-bit hash of the host identity (boot id).  Both ends must agree:
//         the transport is intra-node.
//   qp_n  process id of the endpoint's owner.
//   psn   random nonce.  (qp_n, psn) names the shared-memory inbox
//         "/ibcomm.<qp_n>.<psn>" and the abstract unix socket of the same
//         name that hands out file descriptors of device allocations.
#pragma once

#include <cstdint>

struct ProcessInfo {
  uint16_t lid;
  uint32_t qp_n;
  uint32_t psn;
};
