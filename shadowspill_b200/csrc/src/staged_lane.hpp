// File-backed spill pool and the staged lanes that move bytes between it and the
// device pool.
//
// A transfer is cut into chunks. Each chunk passes through one slot of a bounded ring
// of pinned host memory: for a fetch a disk thread reads the chunk from the file into
// the slot and the runtime's worker then enqueues the host-to-device copy; for an
// evict the worker enqueues the device-to-host copy and, once its event has completed,
// a disk thread writes the slot to the file. Disk threads only read and write the file
// and flip slot states; every backend call (copies, events, stream waits) is made by
// the runtime's worker thread inside pump(). The same division is used by the
// reference's SSD extension (packages/engine/csrc/ssd/{pool,lane,lane_io}.c).
//
// The file is opened twice, with and without O_DIRECT. A chunk whose file offset,
// length and buffer are all multiples of 4096 goes through the direct descriptor; any
// other chunk (the ragged tail of an object) and whole-object host I/O use the buffered
// one. Where the filesystem refuses O_DIRECT everything is buffered.
#pragma once
#include "common.hpp"

#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <thread>

namespace ssc {

constexpr int64_t DIRECT_ALIGN = 4096;

// Where a staged lane's chunks live: a local file or memory held by a remote daemon.
class ChunkStore {
 public:
  virtual ~ChunkStore() = default;
  virtual bool is_open() const = 0;
  virtual int64_t bytes() const = 0;
  // Whole-range host I/O (initialisation, checkpoints); complete on return.
  virtual int write(int64_t off, const void* src, int64_t n) = 0;
  virtual int read(int64_t off, void* dst, int64_t n) = 0;
  // One chunk for a lane; called from several disk threads at once.
  virtual int chunk_io(bool write, void* buf, int64_t off, int64_t n) = 0;
};

class FilePool : public ChunkStore {
 public:
  ~FilePool() override { close(); }
  // directory: where the unlinked scratch file lives. image: optional named file.
  // image_mode 0: the image is the whole pool, opened read-write and kept. 1: the same, created
  // here (it must not exist). 2 (adopt): the existing image is opened read-only as the pool's
  // first bytes, the rest of the pool is a scratch file in `directory`; writing into the image
  // part fails.
  int open(const char* directory, const char* image, int image_mode, int64_t bytes,
           std::string& error);
  int64_t image_bytes() const { return image_bytes_; }
  void close();
  bool is_open() const override { return fd_buffered_ >= 0; }
  bool direct() const { return fd_direct_ >= 0; }
  int64_t bytes() const override { return bytes_; }
  // buffered, durable on return
  int write(int64_t off, const void* src, int64_t n) override;
  int read(int64_t off, void* dst, int64_t n) override;
  // picks the direct descriptor when everything is aligned
  int chunk_io(bool write, void* buf, int64_t off, int64_t n) override;

 private:
  int region_io(bool write, bool chunk, char* buf, int64_t off, int64_t n);
  int fd_direct_ = -1, fd_buffered_ = -1;
  int fd_image_ = -1;            // adopt mode: read-only image holding [0, image_bytes_)
  int64_t image_bytes_ = 0;
  int64_t bytes_ = 0;
};

// A region of host memory held by a memory daemon on another machine (or this one),
// reached over TCP. Control and data use one line-oriented protocol:
//   ALLOCATE <bytes>          -> OK <region>        the region lives while this connection does
//   CONNECT <region>          -> OK <bytes>         further data connections of the same client
//   WRITE <offset> <n> + n B  -> OK
//   READ <offset> <n>         -> OK <n> + n B
//   FREE <region>             -> OK
//   STAT                      -> OK <regions> <bytes held>
// Every calling thread borrows a connection from a small pool, so disk threads of both
// lanes stream concurrently. The reference's network extension moves the same chunks with
// one-sided RDMA where a NIC allows and through a staged host ring otherwise
// (packages/engine/csrc/network/src/{remote_memory,remote_lane_staging,control}.c); this is
// the staged form over sockets.
class RemotePool : public ChunkStore {
 public:
  ~RemotePool() override { close(); }
  int open(const char* address, int64_t bytes, std::string& error);   // "host:port"
  void close();
  bool is_open() const override { return control_fd_ >= 0; }
  int64_t bytes() const override { return bytes_; }
  int write(int64_t off, const void* src, int64_t n) override { return chunk_io(true, const_cast<void*>(src), off, n); }
  int read(int64_t off, void* dst, int64_t n) override { return chunk_io(false, dst, off, n); }
  int chunk_io(bool write, void* buf, int64_t off, int64_t n) override;

 private:
  int connect_data();
  int borrow();
  void give_back(int fd);
  std::string host_;
  int port_ = 0;
  int control_fd_ = -1;
  int64_t region_ = -1, bytes_ = 0;
  std::mutex mu_;
  std::vector<int> idle_;
};

struct StagedJob {
  // filled by the submitter
  bool to_device = true;
  int64_t file_off = 0;
  char* dev = nullptr;
  int64_t bytes = 0;
  int32_t tag = -1;                                  // the submitter's action index
  // 0 = waits enqueued, go on; 1 = not yet (the lane retries later); <0 = error
  std::function<int(StagedJob&)> before_first_copy;
  std::function<int(StagedJob&)> after_last_copy;    // record completion events
  std::function<void(StagedJob&)> on_durable;        // evict: every chunk is in the file
  // lane state
  int64_t posted = 0;     // fetch: bytes handed to disk threads; evict: bytes whose copy is enqueued
  int64_t copied = 0;     // fetch: bytes whose copy is enqueued
  std::atomic<int64_t> written{0};                   // evict: bytes written to the file
  bool finished = false;
  void reset() { posted = copied = 0; written.store(0); finished = false; }
};

class StagedLane {
 public:
  StagedLane(ss_backend* be, void* stream, ChunkStore* pool, bool to_device, int64_t chunk_bytes,
             int32_t queue_depth, int32_t io_threads);
  ~StagedLane();
  int init(int numa_node);                 // allocates the ring and starts the disk threads
  void submit(StagedJob* job);             // worker thread only
  // Advances every state machine once. Returns >0 if anything moved, 0 if not, <0 on error
  // (message() says what failed).
  int pump();
  bool busy() const { return !jobs_.empty(); }
  const std::string& message() const { return message_; }
  int64_t ring_bytes() const { return chunk_ * depth_; }
  int64_t chunks_done() const { return chunks_done_.load(std::memory_order_relaxed); }
  int64_t bytes_done() const { return bytes_done_.load(std::memory_order_relaxed); }

 private:
  enum SlotState : int { FREE = 0, READING, FILLED, COPYING, COPIED, WRITING, WRITTEN, FAILED };
  struct Slot {
    char* buf = nullptr;
    void* event = nullptr;
    std::atomic<int> state{FREE};
    StagedJob* job = nullptr;
    int64_t off = 0, n = 0;                 // offset inside the job
  };
  void disk_main();
  int take_free();
  int fail(const char* what);

  ss_backend* be_;
  void* stream_;
  ChunkStore* pool_;
  bool to_device_;
  int64_t chunk_;
  int32_t depth_, io_threads_;
  char* ring_ = nullptr;
  std::vector<Slot> slots_;
  std::deque<StagedJob*> jobs_;             // submitted, not finished; FIFO
  size_t read_cursor_ = 0;                  // fetch: index into jobs_ of the job being read ahead
  std::deque<int> order_;                   // fetch: slots in posting order; evict: slots copying
  std::deque<int> copying_;                 // fetch: slots whose copy is in flight
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<int> disk_queue_;
  std::vector<std::thread> threads_;
  bool stop_ = false;
  std::string message_;
  std::atomic<int64_t> chunks_done_{0}, bytes_done_{0};     // chunks the disk threads completed
};

}  // namespace ssc
