// Stress driver for the host-side native code, built by tests/test_cpu_native_sanitizers.py with
// -fsanitize=address,undefined and with -fsanitize=thread: the serving scheduler / KV block
// allocator under concurrent submitters, the .rrec reader and the multi-threaded batch loader over
// several epochs (including one abandoned half way), and the file-descriptor exchange between ranks.  Exits 0 when every invariant held; the
// sanitizers abort the process on a report.
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>
#include <unistd.h>

extern "C" {
void* rbs_create(int num_blocks, int block_size, int max_batch, int token_budget);
void rbs_destroy(void* h);
int rbs_num_free_blocks(void* h);
int rbs_num_waiting(void* h);
int rbs_num_running(void* h);
long long rbs_num_preemptions(void* h);
int rbs_add_request(void* h, long long id, int prompt_len, int max_new);
int rbs_schedule(void* h, long long* decode_ids, int* n_decode, long long* prefill_ids,
                 int* prefill_start, int* prefill_len, int* n_prefill, int max_out);
int rbs_commit(void* h, const long long* decode_ids, int n_decode, const long long* prefill_ids,
               const int* prefill_len, int n_prefill, const long long* eos_ids, int n_eos,
               long long* finished_ids, int max_out);
int rbs_block_table(void* h, long long id, int* out, int max_blocks);

void* rrec_open(const char* path);
void rrec_close(void* h);
long long rrec_len(void* h);
long long rrec_tensor(void* h, long long idx, int which, int* ndim, int* shape, int* dtype,
                      const void** data);

void* rbl_create(const char* path, int batch, int drop_last, int workers, int slots, void* in_buf,
                 void* tg_buf);
long long rbl_num_batches(void* h);
void rbl_start_epoch(void* h, int do_shuffle);
int rbl_next(void* h, int* rows);
void rbl_release(void* h, int s);
void rbl_destroy(void* h);
}

#define CHECK(c)                                                              \
  do {                                                                        \
    if (!(c)) { std::fprintf(stderr, "CHECK failed: %s (line %d)\n", #c, __LINE__); return 1; } \
  } while (0)

static int scheduler_stress() {
  const int blocks = 48, bs = 8;
  void* s = rbs_create(blocks, bs, 6, 64);
  CHECK(s != nullptr);
  std::atomic<long long> next_id{1};
  std::atomic<int> accepted{0};
  // submitters run while the engine loop schedules: the scheduler's mutex is what is under test
  std::vector<std::thread> subs;
  for (int t = 0; t < 3; ++t)
    subs.emplace_back([&, t] {
      for (int i = 0; i < 40; ++i) {
        const long long id = next_id.fetch_add(1);
        if (rbs_add_request(s, id, 5 + (int)((id * 7 + t) % 40), 3 + (int)(id % 9)) == 0) accepted++;
      }
    });
  int finished = 0, idle = 0;
  std::vector<long long> dec(64), pre(64), fin(64);
  std::vector<int> pst(64), pln(64), table(64);
  while (idle < 2000) {
    int nd = 0, np = 0;
    const int tokens = rbs_schedule(s, dec.data(), &nd, pre.data(), pst.data(), pln.data(), &np, 64);
    if (tokens == 0) { ++idle; std::this_thread::yield(); if (finished == accepted.load() && idle > 200) break; continue; }
    idle = 0;
    CHECK(tokens <= 64 && nd <= 6 + 64);
    for (int i = 0; i < nd; ++i) CHECK(rbs_block_table(s, dec[i], table.data(), 64) > 0);
    const int nf = rbs_commit(s, dec.data(), nd, pre.data(), pln.data(), np, nullptr, 0, fin.data(), 64);
    CHECK(nf >= 0);
    finished += nf;
    CHECK(rbs_num_free_blocks(s) >= 0 && rbs_num_free_blocks(s) <= blocks);
  }
  for (auto& t : subs) t.join();
  // drain what arrived after the loop went idle
  for (int guard = 0; guard < 100000 && finished < accepted.load(); ++guard) {
    int nd = 0, np = 0;
    if (rbs_schedule(s, dec.data(), &nd, pre.data(), pst.data(), pln.data(), &np, 64) == 0) continue;
    finished += rbs_commit(s, dec.data(), nd, pre.data(), pln.data(), np, nullptr, 0, fin.data(), 64);
  }
  CHECK(finished == accepted.load());
  CHECK(rbs_num_free_blocks(s) == blocks && rbs_num_running(s) == 0 && rbs_num_waiting(s) == 0);
  std::printf("scheduler: %d requests, %lld preemptions\n", finished, rbs_num_preemptions(s));
  rbs_destroy(s);
  return 0;
}

static void put32(std::string& o, uint32_t v) { o.append(reinterpret_cast<const char*>(&v), 4); }
static void put64(std::string& o, uint64_t v) { o.append(reinterpret_cast<const char*>(&v), 8); }

static int write_rrec(const char* path, int n, int in_elems, int tg_elems) {
  std::string body(64, '\0');
  std::vector<std::pair<uint64_t, uint64_t>> index;
  for (int r = 0; r < n; ++r) {
    const uint64_t off = body.size();
    put32(body, 1); put32(body, (uint32_t)in_elems); put32(body, 0);
    for (int i = 0; i < in_elems; ++i) { float v = (float)(r * 1000 + i); body.append(reinterpret_cast<const char*>(&v), 4); }
    put32(body, 1); put32(body, (uint32_t)tg_elems); put32(body, 0);
    for (int i = 0; i < tg_elems; ++i) { float v = (float)r; body.append(reinterpret_cast<const char*>(&v), 4); }
    index.emplace_back(off, body.size() - off);
  }
  const uint64_t index_off = body.size();
  for (auto& e : index) { put64(body, e.first); put64(body, e.second); }
  std::string head = "RREC";
  put32(head, 1); put64(head, (uint64_t)n); put64(head, index_off);
  std::memcpy(&body[0], head.data(), head.size());
  FILE* f = std::fopen(path, "wb");
  if (!f) return 1;
  std::fwrite(body.data(), 1, body.size(), f);
  std::fclose(f);
  return 0;
}

static int loader_stress(const char* path) {
  const int n = 53, in_elems = 12, tg_elems = 3, batch = 8, slots = 3;
  CHECK(write_rrec(path, n, in_elems, tg_elems) == 0);
  void* r = rrec_open(path);
  CHECK(r != nullptr && rrec_len(r) == n);
  int ndim, shape[8], dtype;
  const void* data;
  CHECK(rrec_tensor(r, n - 1, 1, &ndim, shape, &dtype, &data) == tg_elems * 4);
  CHECK(rrec_tensor(r, n, 0, &ndim, shape, &dtype, &data) == -1);
  rrec_close(r);
  std::vector<float> in_ring((size_t)slots * batch * in_elems), tg_ring((size_t)slots * batch * tg_elems);
  void* L = rbl_create(path, batch, 0, 4, slots, in_ring.data(), tg_ring.data());
  CHECK(L != nullptr && rbl_num_batches(L) == (n + batch - 1) / batch);
  for (int epoch = 0; epoch < 4; ++epoch) {
    rbl_start_epoch(L, epoch % 2);
    std::vector<int> seen(n, 0);
    int taken = 0;
    for (;;) {
      int rows = 0;
      const int s = rbl_next(L, &rows);
      if (s == -1) break;
      CHECK(s >= 0 && rows > 0 && rows <= batch);
      for (int i = 0; i < rows; ++i) {
        const int rec = (int)tg_ring[((size_t)s * batch + i) * tg_elems];
        CHECK(rec >= 0 && rec < n);
        CHECK(in_ring[((size_t)s * batch + i) * in_elems + 5] == (float)(rec * 1000 + 5));
        seen[rec]++;
      }
      rbl_release(L, s);
      ++taken;
      if (epoch == 2 && taken == 2) break;   // abandon this epoch half way
    }
    if (epoch != 2)
      for (int i = 0; i < n; ++i) CHECK(seen[i] == 1);
  }
  rbl_destroy(L);
  std::printf("loader: ok\n");
  return 0;
}

extern "C" int rb_fd_exchange(const char* dir, int rank, int world, int my_fd, int* out_fds, int timeout_ms);

// Four "ranks" (threads; descriptors pass through real Unix sockets all the same) exchange the read
// ends of pipes; every rank then finds every other rank's byte in the pipe it received.
static int fd_exchange_stress(const std::string& dir) {
  const int world = 4;
  for (int round = 0; round < 3; ++round) {
    int pipes[world][2];
    for (int r = 0; r < world; ++r) {
      CHECK(pipe(pipes[r]) == 0);
      const char b = (char)('a' + r);
      CHECK(write(pipes[r][1], &b, 1) == 1);
    }
    std::vector<std::vector<int>> got(world, std::vector<int>(world, -1));
    std::vector<int> rc(world, -1);
    std::vector<std::thread> th;
    for (int r = 0; r < world; ++r)
      th.emplace_back([&, r] { rc[r] = rb_fd_exchange(dir.c_str(), r, world, pipes[r][0], got[r].data(), 10000); });
    for (auto& t : th) t.join();
    for (int r = 0; r < world; ++r) {
      CHECK(rc[r] == 0);
      for (int p = 0; p < world; ++p) CHECK(got[r][p] >= 0);
      CHECK(got[r][r] == pipes[r][0]);
    }
    // one reader per pipe: rank (p+1)%world reads rank p's byte through the descriptor it received
    for (int p = 0; p < world; ++p) {
      char b = 0;
      CHECK(read(got[(p + 1) % world][p], &b, 1) == 1);
      CHECK(b == (char)('a' + p));
    }
    for (int r = 0; r < world; ++r) {
      for (int p = 0; p < world; ++p) if (p != r) close(got[r][p]);
      close(pipes[r][0]);
      close(pipes[r][1]);
    }
  }
  std::printf("fd exchange: ok\n");
  return 0;
}

int main(int argc, char** argv) {
  if (argc < 2) { std::fprintf(stderr, "usage: driver <scratch .rrec path>\n"); return 2; }
  if (scheduler_stress()) return 1;
  if (loader_stress(argv[1])) return 1;
  {
    std::string dir(argv[1]);
    const size_t slash = dir.find_last_of('/');
    if (fd_exchange_stress(slash == std::string::npos ? std::string(".") : dir.substr(0, slash))) return 1;
  }
  std::printf("HOST SANITIZE DRIVER OK\n");
  return 0;
}
