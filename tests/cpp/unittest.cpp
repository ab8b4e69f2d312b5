// Unit tests of the host utilities: the size parser tables and the
// power-of-two gate (cases of the reference's tests/unittest.cpp:12-71, with
// the current function name), the partitioner, the expression compiler and the
// error policy, and the staging pool's lease, order and growth (the contract of
// the reference's memory_pool.h:111-121,222-243).
#include <cstring>

#include "ibcomm/communicator.h"
#include "ibcomm/expr.h"
#include "ibcomm/memory_pool.h"
#include "mini_test.h"

using util::parse_number;

MINI_TEST(ParseNumberZero) {
  for (const char* sign : {"", "-", "+"}) {
    for (const char* suffix : {"", "b", "B", "k", "kb", "K", "KB", "m", "mb", "M", "g", "gb", "G"}) {
      std::string s = std::string(sign) + "0" + suffix;
      CHECK_EQ(parse_number(s), int64_t(0));
    }
  }
}

MINI_TEST(ParseNumberPositive) {
  CHECK_EQ(parse_number("1"), int64_t(1));
  CHECK_EQ(parse_number("1b"), int64_t(1));
  CHECK_EQ(parse_number("1B"), int64_t(1));
  CHECK_EQ(parse_number("1k"), int64_t(1024));
  CHECK_EQ(parse_number("1kb"), int64_t(1024));
  CHECK_EQ(parse_number("31k"), int64_t(31 * 1024));
  CHECK_EQ(parse_number("31kb"), int64_t(31 * 1024));
  CHECK_EQ(parse_number("713m"), int64_t(713) * 1024 * 1024);
  CHECK_EQ(parse_number("713mb"), int64_t(713) * 1024 * 1024);
  CHECK_EQ(parse_number("128M"), int64_t(128) << 20);
  CHECK_EQ(parse_number("2g"), int64_t(2) << 30);
  CHECK_EQ(parse_number("-128"), int64_t(-128));
  CHECK_EQ(parse_number("-3K"), int64_t(-3072));
}

MINI_TEST(ParseNumberMalformed) {
  for (const char* s : {"0.5", "a", "b", "B", "0x", "97MiB", "", "-", "k", "1kk", "1 k", "12bb", "9999999999999999999999"})
    CHECK_THROWS(parse_number(s), util::MalformedNumber);
}

MINI_TEST(GetExpOfTwo) {
  CHECK_EQ(util::GetExpOfTwo(0), 0);
  CHECK_EQ(util::GetExpOfTwo(1), 0);
  CHECK_EQ(util::GetExpOfTwo(2), 1);
  CHECK_EQ(util::GetExpOfTwo(128), 7);
  CHECK_EQ(util::GetExpOfTwo(127), 0);
  CHECK_EQ(util::GetExpOfTwo(129), 0);
  CHECK_EQ(util::GetExpOfTwo(uint64_t(1) << 40), 40);
  CHECK_EQ(util::FloorPow2(1), uint64_t(1));
  CHECK_EQ(util::FloorPow2(7), uint64_t(4));
  CHECK_EQ(util::FloorPow2(8), uint64_t(8));
  CHECK_EQ(util::ceilDiv(10, 4), 3);
  CHECK_EQ(util::ceilDiv(size_t(8), size_t(4)), size_t(2));
}

MINI_TEST(SplitBufferDefault) {
  // 4 * ws chunks of ceil(n / chunks); contiguous, covering, ordered.
  auto r = ibcomm::SplitBuffer(1000, 4, 4, 0);
  CHECK_EQ(r.size(), size_t(16));
  CHECK_EQ(r.front().first, size_t(0));
  CHECK_EQ(r.back().second, size_t(1000));
  for (size_t i = 1; i < r.size(); ++i) CHECK_EQ(r[i].first, r[i - 1].second);
  CHECK_EQ(r[0].second - r[0].first, size_t(63));
  // Short message: empty tail ranges are dropped (n = 4, ws = 2 -> 4 ranges).
  auto s = ibcomm::SplitBuffer(4, 4, 2, 0);
  CHECK_EQ(s.size(), size_t(4));
  // 64-bit indices survive lengths beyond 2^31 elements.
  auto big = ibcomm::SplitBuffer((size_t(1) << 33) + 5, 4, 8, 0);
  CHECK_EQ(big.back().second, (size_t(1) << 33) + 5);
  CHECK_EQ(big.size(), size_t(32));
}

MINI_TEST(SplitBufferEnvChunk) {
  auto r = ibcomm::SplitBuffer(256, 4, 4, 64);  // 16 elements per chunk
  CHECK_EQ(r.size(), size_t(16));
  CHECK_EQ(r[3].first, size_t(48));
  auto m = ibcomm::GetRankToChunk(r.size(), 4);
  CHECK_EQ(m[0].size(), size_t(4));
  CHECK_EQ(m[1][0], 4);
  CHECK_EQ(m[3][3], 15);
  auto odd = ibcomm::GetRankToChunk(10, 4);  // 3 3 2 2
  CHECK_EQ(odd[0].size(), size_t(3));
  CHECK_EQ(odd[1].size(), size_t(3));
  CHECK_EQ(odd[2].size(), size_t(2));
  CHECK_EQ(odd[3][1], 9);
}

MINI_TEST(SplitBufferErrors) {
  ibcomm::SetErrorPolicy(ibcomm::ErrorPolicy::kThrow);
  auto code = [](auto fn) {
    try {
      fn();
    } catch (const ibcomm::Error& e) {
      return e.code();
    }
    return 0;
  };
  CHECK_EQ(code([] { ibcomm::SplitBuffer(1, 4, 2, 0); }), 4);        // shorter than world size
  CHECK_EQ(code([] { ibcomm::SplitBuffer(256, 4, 4, 3); }), 1);      // not a multiple of sizeof(T)
  CHECK_EQ(code([] { ibcomm::SplitBuffer(256, 4, 4, 1024); }), 1);   // fewer than 2 * ws chunks
  CHECK_EQ(code([] { ibcomm::SplitBuffer(256, 4, 4, 128); }), 0);    // exactly 2 * ws chunks
  CHECK_EQ(code([] { ibcomm::SplitBuffer(1, 4, 2, 3); }), 4);        // length is checked first
  ibcomm::SetErrorPolicy(ibcomm::ErrorPolicy::kExit);
}

MINI_TEST(SplitEven) {
  auto r = ibcomm::SplitEven(10, 4);
  CHECK_EQ(r.size(), size_t(4));
  CHECK_EQ(r[0].first, size_t(0));
  CHECK_EQ(r[3].second, size_t(10));
  for (size_t i = 1; i < r.size(); ++i) CHECK_EQ(r[i].first, r[i - 1].second);
}

MINI_TEST(Expr) {
  double p = 2, np = 4, n = 8, nb = 32, i = 3;
  std::map<std::string, const double*> vars{{"p", &p}, {"np", &np}, {"n", &n}, {"nb", &nb}, {"i", &i}};
  CHECK_EQ(ibcomm::Expr("i*np+p", vars).Eval(), 14.0);
  CHECK_EQ(ibcomm::Expr("i*np*np+np*(np-1)/2", vars).Eval(), 54.0);
  CHECK_EQ(ibcomm::Expr("1/np*p+i", vars).Eval(), 3.5);
  CHECK_EQ(ibcomm::Expr("-2^2", vars).Eval(), -4.0);
  CHECK_EQ(ibcomm::Expr("2^3^2", vars).Eval(), 512.0);
  CHECK_EQ(ibcomm::Expr("max(p, np) + min(1, 2) + abs(-3) + 7 % 4", vars).Eval(), 11.0);
  CHECK_EQ(ibcomm::Expr(" ( nb ) / n ", vars).Eval(), 4.0);
  i = 5;
  ibcomm::Expr e("i", vars);
  CHECK_EQ(e.Eval(), 5.0);
  i = 6;
  CHECK_EQ(e.Eval(), 6.0);
  CHECK_THROWS(ibcomm::Expr("i +", vars), ibcomm::ExprError);
  CHECK_THROWS(ibcomm::Expr("q", vars), ibcomm::ExprError);
  CHECK_THROWS(ibcomm::Expr("(1", vars), ibcomm::ExprError);
  CHECK_THROWS(ibcomm::Expr("sqrt(1, 2)", vars), ibcomm::ExprError);
}

MINI_TEST(ErrorPolicyThrow) {
  ibcomm::SetErrorPolicy(ibcomm::ErrorPolicy::kThrow);
  int code = 0;
  std::string what;
  try {
    IBCOMM_FAIL(NOT_SUPPORTED, "value %d\n", 7);
  } catch (const ibcomm::Error& e) {
    code = e.code();
    what = e.what();
  }
  CHECK_EQ(code, 4);
  CHECK_TRUE(what.find("Error occured at") == 0);
  CHECK_TRUE(what.find("value 7") != std::string::npos);
  ibcomm::SetErrorPolicy(ibcomm::ErrorPolicy::kExit);
}

MINI_TEST(TraceNull) {
  ibcomm::SetErrorPolicy(ibcomm::ErrorPolicy::kThrow);
  CHECK_THROWS(util::trace(nullptr), ibcomm::Error);
  std::vector<struct timespec> v;
  util::trace(&v);
  CHECK_EQ(v.size(), size_t(1));
  ibcomm::SetErrorPolicy(ibcomm::ErrorPolicy::kExit);
}

MINI_TEST(MemoryPoolLeaseAndOrder) {
  ibcomm::SetErrorPolicy(ibcomm::ErrorPolicy::kThrow);
  ibcomm::MemoryPool<> pool(4096, 2);
  CHECK_EQ(pool.num_blocks(), size_t(1));
  {
    auto c = pool.GetController(1024);
    CHECK_EQ(c.total_slots(), size_t(4));
    int code = 0;
    try {
      auto second = pool.GetController(1024);
    } catch (const ibcomm::Error& e) {
      code = e.code();
    }
    CHECK_EQ(code, 4);  // one controller at a time
    ibcomm::Memory* a = c.getMemory();
    ibcomm::Memory* b = c.getMemory();
    CHECK_EQ(a->offset(), size_t(0));
    CHECK_EQ(b->offset(), size_t(1024));
    CHECK_TRUE(a->stream() != nullptr && b->stream() != nullptr && a->stream() != b->stream());
    // A third slot needs a third stream: the pool creates one.
    ibcomm::Memory* d = c.getMemory();
    CHECK_EQ(pool.num_streams(), size_t(3));
    CHECK_TRUE(d->stream() != a->stream() && d->stream() != b->stream());
    // First in, first out: the slot and the stream that came back first go out after the untouched ones.
    ibcomm::StreamHandle sa = a->stream();
    c.returnMemory(a);
    CHECK_TRUE(a->stream() == nullptr);
    ibcomm::Memory* e = c.getMemory();
    CHECK_EQ(e->offset(), size_t(3072));
    CHECK_TRUE(e->stream() == sa);
    ibcomm::Memory* f = nullptr;
    c.returnMemory(b);
    f = c.getMemory();
    CHECK_TRUE(f == a);
    CHECK_THROWS(c.returnMemory(nullptr), ibcomm::Error);
    std::memset(f->ptr(), 0x5a, 1024);  // the slot is real memory
  }
  CHECK_TRUE(!pool.controller_in_use());
  auto again = pool.GetController(4096);  // released by the destructor
  CHECK_EQ(again.total_slots(), size_t(1));
  ibcomm::SetErrorPolicy(ibcomm::ErrorPolicy::kExit);
}

MINI_TEST(MemoryPoolGrowsAndValidates) {
  ibcomm::SetErrorPolicy(ibcomm::ErrorPolicy::kThrow);
  ibcomm::MemoryPool<> pool(8192, 8);
  auto c = pool.GetController(4096);
  ibcomm::Memory* m[5];
  for (int i = 0; i < 5; ++i) m[i] = c.getMemory();
  CHECK_EQ(pool.num_blocks(), size_t(3));  // 2 slots per block, 5 slots handed out
  CHECK_EQ(c.total_slots(), size_t(6));
  CHECK_TRUE(m[2]->block() != m[0]->block() && m[4]->block() != m[2]->block());
  for (int i = 0; i < 5; ++i) c.returnMemory(m[i]);
  CHECK_EQ(c.vacant_slots(), size_t(6));
  auto moved = std::move(c);  // the lease moves with the controller
  CHECK_TRUE(pool.controller_in_use());
  CHECK_EQ(moved.vacant_slots(), size_t(6));
  CHECK_THROWS(ibcomm::MemoryPool<>(2, 1), ibcomm::Error);
  CHECK_THROWS(ibcomm::MemoryPool<>(4096, 0), ibcomm::Error);
  CHECK_THROWS(ibcomm::MemoryPool<>(4096, 1025), ibcomm::Error);
  ibcomm::MemoryPool<> small(4096, 1);
  CHECK_THROWS(small.GetController(8192), ibcomm::Error);
  CHECK_TRUE(!small.controller_in_use());
  ibcomm::SetErrorPolicy(ibcomm::ErrorPolicy::kExit);
}

int main(int argc, char** argv) { return mini::RunAll(argc > 1 ? argv[1] : nullptr); }
