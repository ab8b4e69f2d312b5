// allreduce_tester — integration-test helper with the reference's command
// line (ibcomm/allreduce_tester.cpp:6-40):
//
//   ibcomm_run -np N allreduce_tester [options] <algorithm> <bytes> <init expr> <check expr>
//
//   <algorithm>  ring | rabenseifner (device runs also: nvls | oneshot | direct | auto)
//   <bytes>      buffer size; suffixes k, m, g (binary) and an optional b
//   <init expr>  every element of the send buffer is set to this expression
//   <check expr> every element of the result must equal this expression
//                (absolute tolerance 1e-12)
//   variables    p = rank, np = number of ranks, n = number of elements,
//                nb = buffer size in bytes, i = element index
//
//   options      --device cpu|cuda|auto   where the buffers live (auto: cuda
//                                         when every rank can have its own GPU)
//                --dtype int|float|double element type (default int)
//                --emulate N              run N ranks inside this one process
//                                         on one GPU (single cooperative kernel)
//                --iters K                repeat the allreduce K times
//                --ranks a,b,...          only the listed ranks of the job take
//                                         part (the others exit with status 0);
//                                         p and np then refer to the subset
//                --op allreduce|reduce_scatter|all_gather
//                                         the collective (default allreduce).  For
//                                         the halves <bytes> is the full buffer
//                                         (np blocks, block p belongs to rank p),
//                                         `i` is the index in the full buffer in
//                                         both expressions, and <algorithm> is
//                                         ring on host buffers, auto | nvls |
//                                         direct on device buffers
//
// The exit status is the number of ranks whose check failed, or one of the
// library's error codes (1 invalid argument, 2 transport, 3 CUDA, 4 not
// supported) when the library terminated the rank.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <iostream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "ibcomm/bootstrap.h"
#include "ibcomm/communicator.h"
#include "ibcomm/expr.h"
#ifdef USE_CUDA
#include <cuda_runtime.h>

#include "ibcomm/emu_world.h"
#endif

namespace {

struct Args {
  std::string device = "auto";
  std::string dtype = "int";
  int emulate = 0;
  int iters = 1;
  std::string op = "allreduce";
  std::vector<int> ranks;  // empty = every rank of the job
  std::string algorithm;
  size_t nbytes = 0;
  std::string init_expr, check_expr;
};

[[noreturn]] void Usage(const char* prog, const std::string& why) {
  if (!why.empty()) std::cerr << "allreduce_tester: " << why << std::endl;
  std::cerr << "usage: " << prog
            << " [--device cpu|cuda|auto] [--dtype int|float|double] [--emulate N] [--iters K]"
               " [--op allreduce|reduce_scatter|all_gather]"
               " <algorithm> <bytes> <init expr> <check expr>"
            << std::endl;
  exit(1);
}

Args ParseArgs(int argc, char** argv) {
  Args a;
  std::vector<std::string> pos;
  for (int i = 1; i < argc; ++i) {
    std::string s = argv[i];
    auto need = [&](const char* name) -> std::string {
      if (i + 1 >= argc) Usage(argv[0], std::string(name) + " needs a value");
      return argv[++i];
    };
    if (s == "--device") a.device = need("--device");
    else if (s == "--dtype") a.dtype = need("--dtype");
    else if (s == "--emulate") a.emulate = atoi(need("--emulate").c_str());
    else if (s == "--iters") a.iters = atoi(need("--iters").c_str());
    else if (s == "--op") a.op = need("--op");
    else if (s == "--ranks") {
      std::stringstream ss(need("--ranks"));
      std::string item;
      while (std::getline(ss, item, ',')) a.ranks.push_back(atoi(item.c_str()));
    }
    else pos.push_back(s);
  }
  if (pos.size() != 4) Usage(argv[0], "four positional arguments expected");
  a.algorithm = pos[0];
  try {
    int64_t v = util::parse_number(pos[1]);
    if (v < 0) Usage(argv[0], "negative buffer size");
    a.nbytes = static_cast<size_t>(v);
  } catch (const util::MalformedNumber& e) {
    Usage(argv[0], e.what());
  }
  a.init_expr = pos[2];
  a.check_expr = pos[3];
  if (a.iters < 1) a.iters = 1;
  if (a.op != "allreduce" && a.op != "reduce_scatter" && a.op != "all_gather") Usage(argv[0], "unknown --op " + a.op);
  return a;
}

struct Vars {
  double p = 0, np = 1, n = 0, nb = 0, i = 0;
  std::map<std::string, const double*> Map() const {
    return {{"p", &p}, {"np", &np}, {"n", &n}, {"nb", &nb}, {"i", &i}};
  }
};

// `first` = index of buf[0] in the full buffer (the halves work on one block of it).
template <typename T>
void Fill(std::vector<T>* buf, const std::string& expr_text, Vars* v, size_t first = 0) {
  ibcomm::Expr expr(expr_text, v->Map());
  for (size_t i = 0; i < buf->size(); ++i) {
    v->i = static_cast<double>(first + i);
    (*buf)[i] = static_cast<T>(expr.Eval());
  }
}

template <typename T>
std::vector<std::string> Check(const std::vector<T>& buf, const std::string& expr_text, Vars* v, size_t first = 0) {
  constexpr double eps = 1e-12;
  std::vector<std::string> msgs;
  ibcomm::Expr expr(expr_text, v->Map());
  for (size_t i = 0; i < buf.size(); ++i) {
    v->i = static_cast<double>(first + i);
    const double want = expr.Eval();
    const double got = static_cast<double>(buf[i]);
    if (!(std::fabs(got - want) <= eps)) {
      if (msgs.size() < 1000) {
        std::ostringstream ss;
        ss << "Error: Element [" << first + i << "] must be " << want << " but actually is " << got;
        msgs.push_back(ss.str());
      } else {
        msgs.push_back(std::string());
        break;
      }
    }
  }
  return msgs;
}

template <typename T>
ibcomm::DType DTypeOf();
template <> ibcomm::DType DTypeOf<int>() { return ibcomm::DType::kInt32; }
template <> ibcomm::DType DTypeOf<float>() { return ibcomm::DType::kFloat32; }
template <> ibcomm::DType DTypeOf<double>() { return ibcomm::DType::kFloat64; }

template <typename T>
void RunHost(ibcomm::Communicator* comm, const std::string& algo, const std::vector<T>& in, std::vector<T>* out) {
  if (algo == "ring") comm->AllreduceRing(in.data(), out->data(), in.size());
  else if (algo == "rabenseifner") comm->AllreduceRabenseifner(in.data(), out->data(), in.size());
  else IBCOMM_FAIL(INVALID_ARGUMENT, "Algorithm '%s' is not available for host buffers.\n", algo.c_str());
}

// The halves on host buffers (a ring over the host transport).
template <typename T>
void RunHostHalf(ibcomm::Communicator* comm, const Args& a, const std::vector<T>& in, std::vector<T>* out, size_t block) {
  if (a.algorithm != "ring") IBCOMM_FAIL(INVALID_ARGUMENT, "Host reduce-scatter / all-gather run the ring algorithm.\n");
  if (a.op == "reduce_scatter") comm->ReduceScatter(in.data(), out->data(), block);
  else comm->AllGather(in.data(), out->data(), block);
}

#ifdef USE_CUDA
template <typename T>
void RunDeviceHalf(ibcomm::Communicator* comm, const Args& a, const std::vector<T>& in, std::vector<T>* out, size_t block) {
  T *d_in = nullptr, *d_out = nullptr;
  CUDACHECK(cudaMalloc(&d_in, std::max<size_t>(in.size() * sizeof(T), 16)));
  CUDACHECK(cudaMalloc(&d_out, std::max<size_t>(out->size() * sizeof(T), 16)));
  CUDACHECK(cudaMemcpy(d_in, in.data(), in.size() * sizeof(T), cudaMemcpyHostToDevice));
  ibcomm::CudaAllreduceOptions o;
  o.algo = ibcomm::AlgoFromName(a.algorithm);
  if (a.op == "reduce_scatter") comm->ReduceScatterCuda(DTypeOf<T>(), d_in, d_out, block, o);
  else comm->AllGatherCuda(DTypeOf<T>(), d_in, d_out, block, o);
  CUDACHECK(cudaMemcpy(out->data(), d_out, out->size() * sizeof(T), cudaMemcpyDeviceToHost));
  CUDACHECK(cudaFree(d_in));
  CUDACHECK(cudaFree(d_out));
}

template <typename T>
void RunDevice(ibcomm::Communicator* comm, const std::string& algo, const std::vector<T>& in, std::vector<T>* out) {
  T *d_in = nullptr, *d_out = nullptr;
  const size_t bytes = in.size() * sizeof(T);
  CUDACHECK(cudaMalloc(&d_in, std::max<size_t>(bytes, 16)));
  CUDACHECK(cudaMalloc(&d_out, std::max<size_t>(bytes, 16)));
  CUDACHECK(cudaMemcpy(d_in, in.data(), bytes, cudaMemcpyHostToDevice));
  if (algo == "ring") {
    comm->AllreduceRingCuda(d_in, d_out, in.size());
  } else if (algo == "rabenseifner") {
    comm->AllreduceRabenseifnerCuda(d_in, d_out, in.size());
  } else {
    ibcomm::CudaAllreduceOptions o;
    o.algo = ibcomm::AlgoFromName(algo);
    comm->AllreduceCuda(DTypeOf<T>(), d_in, d_out, in.size(), o);
  }
  CUDACHECK(cudaMemcpy(out->data(), d_out, bytes, cudaMemcpyDeviceToHost));
  CUDACHECK(cudaFree(d_in));
  CUDACHECK(cudaFree(d_out));
}
#endif

template <typename T>
int RunRanks(const Args& a) {
  ibcomm::BootstrapEnv benv = ibcomm::ReadBootstrapEnv();
  const size_t n = a.nbytes / sizeof(T);

#ifdef USE_CUDA
  if (a.emulate > 0 && a.op != "allreduce")
    IBCOMM_FAIL(NOT_SUPPORTED, "--emulate runs allreduce only.\n");
  if (a.emulate > 0) {
    // All ranks in this process, one GPU, one cooperative kernel.
    const int np = a.emulate;
    std::vector<std::vector<T>> ins(static_cast<size_t>(np), std::vector<T>(n)), outs = ins;
    for (int p = 0; p < np; ++p) {
      Vars v;
      v.p = p; v.np = np; v.n = static_cast<double>(n); v.nb = static_cast<double>(a.nbytes);
      Fill(&ins[static_cast<size_t>(p)], a.init_expr, &v);
    }
    ibcomm::EmuWorld world(np);
    std::vector<const void*> inp;
    std::vector<void*> outp;
    for (int p = 0; p < np; ++p) {
      inp.push_back(ins[static_cast<size_t>(p)].data());
      outp.push_back(outs[static_cast<size_t>(p)].data());
    }
    for (int k = 0; k < a.iters; ++k)
      world.AllreduceHostBuffers(ibcomm::AlgoFromName(a.algorithm), DTypeOf<T>(), inp, outp, n);
    int failed = 0;
    for (int p = 0; p < np; ++p) {
      Vars v;
      v.p = p; v.np = np; v.n = static_cast<double>(n); v.nb = static_cast<double>(a.nbytes);
      std::vector<std::string> msgs = Check(outs[static_cast<size_t>(p)], a.check_expr, &v);
      for (const std::string& m : msgs)
        if (!m.empty()) std::cerr << "[Rank " << p << "] " << m << std::endl;
      failed += msgs.empty() ? 0 : 1;
    }
    return failed;
  }
#else
  if (a.emulate > 0) IBCOMM_FAIL(NOT_SUPPORTED, "--emulate needs the CUDA build of the tester.\n");
#endif

  bool use_cuda = false;
#ifdef USE_CUDA
  if (a.device == "cuda") {
    use_cuda = true;
  } else if (a.device == "auto") {
    int ngpu = 0;
    if (cudaGetDeviceCount(&ngpu) != cudaSuccess) {
      ngpu = 0;
      (void)cudaGetLastError();
    }
    use_cuda = ngpu >= benv.world_size;
  }
  if (use_cuda) {
    int ngpu = 0;
    CUDACHECK(cudaGetDeviceCount(&ngpu));
    if (ngpu < benv.world_size)
      IBCOMM_FAIL(NOT_SUPPORTED,
                  "%d ranks need %d GPUs but %d are visible: ranks that wait on one another must "
                  "not share a GPU. Use --emulate %d instead.\n",
                  benv.world_size, benv.world_size, ngpu, benv.world_size);
    CUDACHECK(cudaSetDevice(benv.local_rank % ngpu));
  }
#else
  if (a.device == "cuda") IBCOMM_FAIL(NOT_SUPPORTED, "This tester was built without CUDA.\n");
#endif

  std::string tag = "c0";
  if (!a.ranks.empty()) {
    if (std::find(a.ranks.begin(), a.ranks.end(), benv.rank) == a.ranks.end()) return 0;  // not a member
    benv = ibcomm::SubsetEnv(benv, a.ranks, &tag);
  }
  ibcomm::Communicator comm(benv.world_size);
  ibcomm::ConnectAll(&comm, benv, tag);

  Vars v;
  v.p = benv.rank;
  v.np = benv.world_size;
  v.n = static_cast<double>(n);
  v.nb = static_cast<double>(a.nbytes);
  // The halves: block `rank` of the full buffer is this rank's.
  const bool half = a.op != "allreduce";
  const size_t np = static_cast<size_t>(benv.world_size);
  if (half && (n == 0 || n % np != 0))
    IBCOMM_FAIL(INVALID_ARGUMENT, "The buffer of %zu elements does not split into %zu equal blocks.\n", n, np);
  const size_t block = half ? n / np : n;
  const size_t mine = half ? block * static_cast<size_t>(benv.rank) : 0;
  const bool rs = a.op == "reduce_scatter", ag = a.op == "all_gather";
  std::vector<T> in(ag ? block : n), out(rs ? block : n);
  Fill(&in, a.init_expr, &v, ag ? mine : 0);

  for (int k = 0; k < a.iters; ++k) {
    if (use_cuda) {
#ifdef USE_CUDA
      if (half) RunDeviceHalf(&comm, a, in, &out, block);
      else RunDevice(&comm, a.algorithm, in, &out);
#endif
    } else {
      if (half) RunHostHalf(&comm, a, in, &out, block);
      else RunHost(&comm, a.algorithm, in, &out);
    }
  }

  std::vector<std::string> msgs = Check(out, a.check_expr, &v, rs ? mine : 0);
  for (int r = 0; r < benv.world_size; ++r) {
    if (r == benv.rank)
      for (const std::string& m : msgs)
        if (!m.empty()) std::cerr << "[Rank " << benv.rank << "] " << m << std::endl;
    comm.Barrier();
  }
  return static_cast<int>(ibcomm::SumOverRanks(&comm, msgs.empty() ? 0 : 1));
}

}  // namespace

int main(int argc, char** argv) {
  Args a = ParseArgs(argc, argv);
  try {
    if (a.dtype == "int") return RunRanks<int>(a);
    if (a.dtype == "float") return RunRanks<float>(a);
    if (a.dtype == "double") return RunRanks<double>(a);
  } catch (const ibcomm::ExprError& e) {
    std::cerr << e.what() << std::endl;
    return 1;
  }
  Usage(argv[0], "unknown --dtype " + a.dtype);
}
