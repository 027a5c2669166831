// Native batch loader over a memory-mapped `.rrec` file (C ABI, loaded with ctypes).
//
// Worker threads assemble whole batches (inputs and targets of `batch` records, copied back to back)
// into a ring of host buffers that the caller provides (pinned memory, so the training loop can
// issue an asynchronous host-to-device copy straight from a slot); the consumer takes batches in
// order.  Epoch order is the reference's Fisher-Yates shuffle driven by its 64-bit LCG
// (rumus/src/data/dataloader.rs:254-274), so a Python `DataLoader(shuffle=True)` over the same file
// visits the records in the same order.
//
// The reference's loader is a feeder thread + worker threads + bounded channels in Rust
// (rumus/src/data/dataloader.rs:16-235); this is its native counterpart for fixed-shape records.
//
// All records must have the same input / target byte sizes (token windows, fixed-size images);
// rbl_create refuses a file where they differ.
#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

extern "C" {
void* rrec_open(const char* path);
void rrec_close(void* h);
long long rrec_len(void* h);
long long rrec_tensor(void* h, long long idx, int which, int* ndim, int* shape, int* dtype,
                      const void** data);
}

namespace {

struct Lcg {
  uint64_t s;
  uint64_t next() {
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    return s;
  }
};

struct Slot {
  int state = 0;          // 0 free, 1 being filled, 2 ready
  long long batch = -1;   // batch index held
  int rows = 0;           // records in it (the last batch may be short)
};

struct Loader {
  void* rrec = nullptr;
  long long n = 0;
  int batch = 0, drop_last = 0, slots = 0;
  long long in_bytes = 0, tg_bytes = 0;
  uint8_t* in_buf = nullptr;   // [slots][batch][in_bytes]
  uint8_t* tg_buf = nullptr;   // [slots][batch][tg_bytes]
  std::vector<long long> order;
  long long num_batches = 0;
  long long next_to_fill = 0;   // next batch index a worker may claim
  long long next_to_take = 0;   // next batch index the consumer returns
  std::vector<Slot> slot;
  std::mutex mu;
  std::condition_variable cv_free, cv_ready;
  std::vector<std::thread> workers;
  bool stop = false;
  Lcg rng{0xDEADBEEFCAFE1234ull};
  int error = 0;
};

void shuffle(Loader* L) {
  for (long long i = L->n - 1; i > 0; --i) {
    const long long j = (long long)(L->rng.next() % (uint64_t)(i + 1));
    std::swap(L->order[i], L->order[j]);
  }
}

void work(Loader* L) {
  for (;;) {
    long long b;
    int s;
    {
      std::unique_lock<std::mutex> lk(L->mu);
      for (;;) {
        if (L->stop) return;
        if (L->next_to_fill < L->num_batches) {
          // a batch may only go into its ring slot once the batch that used it was taken
          b = L->next_to_fill;
          s = (int)(b % L->slots);
          if (L->slot[s].state == 0) break;
        }
        L->cv_free.wait(lk);
      }
      L->next_to_fill++;
      L->slot[s].state = 1;
      L->slot[s].batch = b;
    }
    const long long r0 = b * L->batch;
    const long long r1 = std::min<long long>(L->n, r0 + L->batch);
    int bad = 0;
    for (long long r = r0; r < r1; ++r) {
      int ndim, shape[8], dtype;
      const void* data = nullptr;
      const long long idx = L->order[r];
      long long sz = rrec_tensor(L->rrec, idx, 0, &ndim, shape, &dtype, &data);
      if (sz != L->in_bytes) { bad = 1; break; }
      std::memcpy(L->in_buf + ((size_t)s * L->batch + (size_t)(r - r0)) * L->in_bytes, data, (size_t)sz);
      sz = rrec_tensor(L->rrec, idx, 1, &ndim, shape, &dtype, &data);
      if (sz != L->tg_bytes) { bad = 1; break; }
      std::memcpy(L->tg_buf + ((size_t)s * L->batch + (size_t)(r - r0)) * L->tg_bytes, data, (size_t)sz);
    }
    {
      std::lock_guard<std::mutex> lk(L->mu);
      if (bad) L->error = 1;
      L->slot[s].rows = (int)(r1 - r0);
      L->slot[s].state = 2;
    }
    L->cv_ready.notify_all();
  }
}

void start_epoch(Loader* L, int do_shuffle) {
  for (long long i = 0; i < L->n; ++i) L->order[i] = i;
  if (do_shuffle) shuffle(L);
  L->next_to_fill = 0;
  L->next_to_take = 0;
  for (auto& s : L->slot) s = Slot{};
}

}  // namespace

extern "C" {

// Record sizes of record 0 (bytes) and its shapes / dtypes, so the caller can size the ring.
int rbl_probe(const char* path, long long* n, long long* in_bytes, long long* tg_bytes, int* in_ndim,
              int* in_shape, int* in_dtype, int* tg_ndim, int* tg_shape, int* tg_dtype) {
  void* r = rrec_open(path);
  if (!r) return 1;
  *n = rrec_len(r);
  const void* d;
  *in_bytes = *n > 0 ? rrec_tensor(r, 0, 0, in_ndim, in_shape, in_dtype, &d) : 0;
  *tg_bytes = *n > 0 ? rrec_tensor(r, 0, 1, tg_ndim, tg_shape, tg_dtype, &d) : 0;
  rrec_close(r);
  return (*in_bytes < 0 || *tg_bytes < 0) ? 2 : 0;
}

// in_buf / tg_buf: caller-owned rings of `slots` batches (slots * batch * record bytes each).
void* rbl_create(const char* path, int batch, int drop_last, int workers, int slots, void* in_buf,
                 void* tg_buf) {
  if (batch <= 0 || workers <= 0 || slots <= 0) return nullptr;
  Loader* L = new Loader;
  L->rrec = rrec_open(path);
  if (!L->rrec) { delete L; return nullptr; }
  L->n = rrec_len(L->rrec);
  L->batch = batch; L->drop_last = drop_last; L->slots = slots;
  int ndim, shape[8], dtype;
  const void* d;
  L->in_bytes = L->n > 0 ? rrec_tensor(L->rrec, 0, 0, &ndim, shape, &dtype, &d) : 0;
  L->tg_bytes = L->n > 0 ? rrec_tensor(L->rrec, 0, 1, &ndim, shape, &dtype, &d) : 0;
  if (L->in_bytes < 0 || L->tg_bytes < 0) { rrec_close(L->rrec); delete L; return nullptr; }
  L->in_buf = static_cast<uint8_t*>(in_buf);
  L->tg_buf = static_cast<uint8_t*>(tg_buf);
  L->order.resize((size_t)L->n);
  L->num_batches = drop_last ? L->n / batch : (L->n + batch - 1) / batch;
  L->slot.resize((size_t)slots);
  L->next_to_fill = L->num_batches;   // idle until the first rbl_start_epoch
  for (int i = 0; i < workers; ++i) L->workers.emplace_back(work, L);
  return L;
}

long long rbl_num_batches(void* h) { return static_cast<Loader*>(h)->num_batches; }

// Begins a new epoch (all batches of the previous one must have been taken or are discarded).
void rbl_start_epoch(void* h, int do_shuffle) {
  Loader* L = static_cast<Loader*>(h);
  {
    std::unique_lock<std::mutex> lk(L->mu);
    // let in-flight fills finish so no worker writes into a slot we are about to reset
    L->next_to_fill = L->num_batches;
    L->cv_ready.wait(lk, [&] {
      for (auto& s : L->slot) if (s.state == 1) return false;
      return true;
    });
    start_epoch(L, do_shuffle);
  }
  L->cv_free.notify_all();
}

// Blocks until the next batch (in order) is ready.  Returns its ring slot (>= 0) and the number of
// records in it, -1 at the end of the epoch, -2 if a record did not have the expected size.
int rbl_next(void* h, int* rows) {
  Loader* L = static_cast<Loader*>(h);
  std::unique_lock<std::mutex> lk(L->mu);
  if (L->next_to_take >= L->num_batches) return -1;
  const long long b = L->next_to_take;
  const int s = (int)(b % L->slots);
  L->cv_ready.wait(lk, [&] { return L->slot[s].state == 2 && L->slot[s].batch == b; });
  if (L->error) return -2;
  *rows = L->slot[s].rows;
  return s;
}

// Hands the slot returned by the last rbl_next back to the workers.
void rbl_release(void* h, int s) {
  Loader* L = static_cast<Loader*>(h);
  {
    std::lock_guard<std::mutex> lk(L->mu);
    L->slot[(size_t)s].state = 0;
    L->next_to_take++;
  }
  L->cv_free.notify_all();
}

void rbl_destroy(void* h) {
  Loader* L = static_cast<Loader*>(h);
  if (!L) return;
  {
    std::lock_guard<std::mutex> lk(L->mu);
    L->stop = true;
  }
  L->cv_free.notify_all();
  for (auto& t : L->workers) t.join();
  rrec_close(L->rrec);
  delete L;
}
}
