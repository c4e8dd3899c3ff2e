// File pool and staged lanes: see staged_lane.hpp for the protocol.
#include "staged_lane.hpp"

#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

namespace ssc {

// ------------------------------------------------------------------ FilePool
int FilePool::open(const char* directory, const char* image, int image_mode, int64_t bytes,
                   std::string& error) {
  close();
  if (bytes <= 0) { error = "file pool needs a positive size"; return SS_INVALID_ARGUMENT; }
  const bool named = image && *image;
  const bool adopt = named && image_mode == 2;
  int64_t scratch_bytes = bytes;
  if (adopt) {
    fd_image_ = ::open(image, O_RDONLY | O_CLOEXEC);
    if (fd_image_ < 0) { error = std::string("cannot open pool image ") + image + ": " + std::strerror(errno); return SS_IO_ERROR; }
    struct stat ist{};
    if (::fstat(fd_image_, &ist) != 0 || ist.st_size <= 0 || ist.st_size % DIRECT_ALIGN != 0 || ist.st_size > bytes) {
      error = "an adopted image is a positive multiple of 4096 bytes, no larger than the pool";
      close();
      return SS_INVALID_ARGUMENT;
    }
    image_bytes_ = ist.st_size;
    scratch_bytes = std::max<int64_t>(bytes - image_bytes_, DIRECT_ALIGN);
  }
  int fd = -1;
  if (named && !adopt) {
    fd = ::open(image, O_RDWR | O_CLOEXEC | (image_mode == 1 ? (O_CREAT | O_EXCL) : 0), 0600);
    if (fd < 0) { error = std::string("cannot open pool image ") + image + ": " + std::strerror(errno); return SS_IO_ERROR; }
  } else {
    if (!directory || !*directory) { error = "file pool needs a directory"; close(); return SS_INVALID_ARGUMENT; }
#ifdef O_TMPFILE
    fd = ::open(directory, O_TMPFILE | O_RDWR | O_CLOEXEC, 0600);
#endif
    if (fd < 0) {             // filesystems without O_TMPFILE: a named file, unlinked at once
      std::string tmpl = std::string(directory) + "/ss_pool_XXXXXX";
      std::vector<char> path(tmpl.begin(), tmpl.end());
      path.push_back('\0');
      fd = ::mkstemp(path.data());
      if (fd >= 0) ::unlink(path.data());
    }
    if (fd < 0) { error = std::string("cannot create a pool file in ") + directory + ": " + std::strerror(errno); close(); return SS_IO_ERROR; }
  }
  struct stat st{};
  if (::fstat(fd, &st) != 0) { error = "fstat failed"; ::close(fd); close(); return SS_IO_ERROR; }
  if (st.st_size < scratch_bytes) {
    if (::ftruncate(fd, scratch_bytes) != 0) {
      error = std::string("cannot size the pool file: ") + std::strerror(errno);
      ::close(fd);
      close();
      return SS_IO_ERROR;
    }
    // reserve the blocks now so that a full disk shows at open, not in the middle of a step;
    // filesystems without preallocation keep the sparse file (the raw call, not the library
    // emulation that would write every block of a multi-GiB pool)
    int rc = ::fallocate(fd, 0, 0, scratch_bytes) == 0 ? 0 : errno;
    if (rc == ENOSPC) {
      error = "not enough space for the pool file";
      ::close(fd);
      close();
      return SS_OUT_OF_MEMORY;
    }
  }
  fd_buffered_ = fd;
  bytes_ = bytes;
  char link[64];
  std::snprintf(link, sizeof link, "/proc/self/fd/%d", fd);
  fd_direct_ = ::open(link, O_RDWR | O_DIRECT | O_CLOEXEC);   // -1 where direct I/O is refused
  return SS_OK;
}

void FilePool::close() {
  if (fd_direct_ >= 0) ::close(fd_direct_);
  if (fd_buffered_ >= 0) ::close(fd_buffered_);
  if (fd_image_ >= 0) ::close(fd_image_);
  fd_direct_ = fd_buffered_ = fd_image_ = -1;
  bytes_ = image_bytes_ = 0;
}

static int full_io(int fd, bool write, char* buf, int64_t off, int64_t n) {
  while (n > 0) {
    ssize_t k = write ? ::pwrite(fd, buf, static_cast<size_t>(n), off)
                      : ::pread(fd, buf, static_cast<size_t>(n), off);
    if (k < 0) {
      if (errno == EINTR) continue;
      return -errno;
    }
    if (k == 0) return -EIO;      // read past the end: the file is sized at open
    buf += k; off += k; n -= k;
  }
  return 0;
}

// One range of the pool: the adopted image serves [0, image_bytes_) read-only, the scratch (or
// whole-pool) file the rest, at offsets counted from the end of the image.
int FilePool::region_io(bool write, bool chunk, char* buf, int64_t off, int64_t n) {
  if (fd_buffered_ < 0 || off < 0 || n < 0 || off + n > bytes_) return SS_INVALID_ARGUMENT;
  if (off < image_bytes_) {
    if (write) return SS_IO_ERROR;                 // the image is never written
    const int64_t k = std::min(n, image_bytes_ - off);
    if (full_io(fd_image_, false, buf, off, k) != 0) return SS_IO_ERROR;
    buf += k; off += k; n -= k;
    if (n == 0) return SS_OK;
  }
  off -= image_bytes_;
  const bool aligned = chunk && fd_direct_ >= 0 && off % DIRECT_ALIGN == 0 && n % DIRECT_ALIGN == 0 &&
                       reinterpret_cast<uintptr_t>(buf) % DIRECT_ALIGN == 0;
  if (aligned) {
    int rc = full_io(fd_direct_, write, buf, off, n);
    if (rc == 0) return SS_OK;
    if (rc != -EINVAL) return SS_IO_ERROR;      // EINVAL: this filesystem wants a coarser alignment
  }
  if (full_io(fd_buffered_, write, buf, off, n) != 0) return SS_IO_ERROR;
  if (write && !chunk && ::fdatasync(fd_buffered_) != 0) return SS_IO_ERROR;
  // leave no cached pages behind: they would grow by the whole pool, and the direct descriptor
  // must not disagree with them
  ::posix_fadvise(fd_buffered_, off, n, POSIX_FADV_DONTNEED);
  return SS_OK;
}

int FilePool::write(int64_t off, const void* src, int64_t n) {
  return region_io(true, false, static_cast<char*>(const_cast<void*>(src)), off, n);
}

int FilePool::read(int64_t off, void* dst, int64_t n) {
  return region_io(false, false, static_cast<char*>(dst), off, n);
}

int FilePool::chunk_io(bool write, void* buf, int64_t off, int64_t n) {
  return region_io(write, true, static_cast<char*>(buf), off, n);
}

// ------------------------------------------------------------------ StagedLane
StagedLane::StagedLane(ss_backend* be, void* stream, ChunkStore* pool, bool to_device,
                       int64_t chunk_bytes, int32_t queue_depth, int32_t io_threads)
    : be_(be), stream_(stream), pool_(pool), to_device_(to_device), chunk_(chunk_bytes),
      depth_(queue_depth), io_threads_(std::max(1, io_threads)), slots_(static_cast<size_t>(queue_depth)) {}

int StagedLane::init(int numa_node) {
  if (chunk_ <= 0 || chunk_ % DIRECT_ALIGN != 0 || depth_ < 1) return SS_INVALID_ARGUMENT;
  void* p = nullptr;
  int rc = be_->host_alloc(be_->self, static_cast<size_t>(chunk_ * depth_), numa_node, &p);
  if (rc != SS_OK) return rc;
  ring_ = static_cast<char*>(p);
  for (int32_t i = 0; i < depth_; ++i) {
    slots_[i].buf = ring_ + static_cast<int64_t>(i) * chunk_;
    rc = be_->event_create(be_->self, 0, &slots_[i].event);
    if (rc != SS_OK) return rc;
  }
  for (int32_t i = 0; i < io_threads_; ++i) threads_.emplace_back([this] { disk_main(); });
  return SS_OK;
}

StagedLane::~StagedLane() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  for (auto& t : threads_) if (t.joinable()) t.join();
  for (auto& s : slots_) if (s.event) be_->event_destroy(be_->self, s.event);
  if (ring_) be_->host_free(be_->self, ring_, static_cast<size_t>(chunk_ * depth_));
}

// Disk threads: file I/O and slot state only.
void StagedLane::disk_main() {
  for (;;) {
    int si;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait(lk, [this] { return stop_ || !disk_queue_.empty(); });
      if (stop_) return;
      si = disk_queue_.front();
      disk_queue_.pop_front();
    }
    Slot& s = slots_[si];
    const int rc = pool_->chunk_io(!to_device_, s.buf, s.job->file_off + s.off, s.n);
    if (rc != SS_OK) { s.state.store(FAILED, std::memory_order_release); continue; }
    chunks_done_.fetch_add(1, std::memory_order_relaxed);
    bytes_done_.fetch_add(s.n, std::memory_order_relaxed);
    if (to_device_) {
      s.state.store(FILLED, std::memory_order_release);
    } else {
      s.job->written.fetch_add(s.n, std::memory_order_acq_rel);
      s.state.store(WRITTEN, std::memory_order_release);
    }
  }
}

int StagedLane::take_free() {
  for (int32_t i = 0; i < depth_; ++i)
    if (slots_[i].state.load(std::memory_order_acquire) == FREE) return i;
  return -1;
}

int StagedLane::fail(const char* what) {
  message_ = what;
  return -1;
}

void StagedLane::submit(StagedJob* job) {
  job->reset();
  jobs_.push_back(job);
}

int StagedLane::pump() {
  int moved = 0;
  ss_backend* be = be_;
  if (to_device_) {
    // 1. slots whose host-to-device copy has completed are free again
    while (!copying_.empty()) {
      Slot& s = slots_[copying_.front()];
      const int rc = be->event_query(be->self, s.event);
      if (rc == SS_TIMEOUT) break;
      if (rc != SS_OK) return fail("slot event failed");
      s.job = nullptr;
      s.state.store(FREE, std::memory_order_release);
      copying_.pop_front();
      ++moved;
    }
    // 2. read ahead, across jobs, into every free slot
    while (read_cursor_ < jobs_.size()) {
      StagedJob* job = jobs_[read_cursor_];
      if (job->posted >= job->bytes) { ++read_cursor_; continue; }
      const int si = take_free();
      if (si < 0) break;
      Slot& s = slots_[si];
      s.job = job; s.off = job->posted; s.n = std::min(chunk_, job->bytes - job->posted);
      job->posted += s.n;
      s.state.store(READING, std::memory_order_release);
      order_.push_back(si);
      {
        std::lock_guard<std::mutex> lk(mu_);
        disk_queue_.push_back(si);
      }
      cv_.notify_one();
      ++moved;
    }
    // 3. filled slots, in posting order, go onto the copy stream
    while (!order_.empty()) {
      const int si = order_.front();
      Slot& s = slots_[si];
      const int st = s.state.load(std::memory_order_acquire);
      if (st == FAILED) return fail("reading the pool file failed");
      if (st != FILLED) break;
      StagedJob* job = s.job;
      if (job->copied == 0 && job->before_first_copy) {
        const int rc = job->before_first_copy(*job);
        if (rc > 0) break;
        if (rc < 0) return fail("stream wait before a staged fetch failed");
      }
      int rc = be->copy_async(be->self, job->dev + s.off, s.buf, static_cast<size_t>(s.n), SS_COPY_H2D, stream_);
      if (rc == SS_OK) rc = be->event_record(be->self, s.event, stream_);
      if (rc != SS_OK) return fail("staged fetch copy failed to enqueue");
      s.state.store(COPYING, std::memory_order_release);
      job->copied += s.n;
      order_.pop_front();
      copying_.push_back(si);
      ++moved;
      if (job->copied == job->bytes) {
        if (job->after_last_copy && job->after_last_copy(*job) != 0) return fail("completion event of a staged fetch failed");
        job->finished = true;
      }
    }
  } else {
    // 1. device-to-host copies that have completed are handed to the disk threads
    while (!order_.empty()) {
      const int si = order_.front();
      Slot& s = slots_[si];
      const int rc = be->event_query(be->self, s.event);
      if (rc == SS_TIMEOUT) break;
      if (rc != SS_OK) return fail("slot event failed");
      s.state.store(WRITING, std::memory_order_release);
      {
        std::lock_guard<std::mutex> lk(mu_);
        disk_queue_.push_back(si);
      }
      cv_.notify_one();
      order_.pop_front();
      ++moved;
    }
    // 2. written slots are free again
    for (auto& s : slots_) {
      const int st = s.state.load(std::memory_order_acquire);
      if (st == FAILED) return fail("writing the pool file failed");
      if (st == WRITTEN) { s.job = nullptr; s.state.store(FREE, std::memory_order_release); ++moved; }
    }
    // 3. enqueue copies, job by job, while slots are free
    while (read_cursor_ < jobs_.size()) {
      StagedJob* job = jobs_[read_cursor_];
      if (job->posted >= job->bytes) { ++read_cursor_; continue; }
      const int si = take_free();
      if (si < 0) break;
      if (job->posted == 0 && job->before_first_copy) {
        const int rc = job->before_first_copy(*job);
        if (rc > 0) break;
        if (rc < 0) return fail("stream wait before a staged evict failed");
      }
      Slot& s = slots_[si];
      s.job = job; s.off = job->posted; s.n = std::min(chunk_, job->bytes - job->posted);
      int rc = be->copy_async(be->self, s.buf, job->dev + s.off, static_cast<size_t>(s.n), SS_COPY_D2H, stream_);
      if (rc == SS_OK) rc = be->event_record(be->self, s.event, stream_);
      if (rc != SS_OK) return fail("staged evict copy failed to enqueue");
      s.state.store(COPYING, std::memory_order_release);
      order_.push_back(si);
      job->posted += s.n;
      ++moved;
      if (job->posted == job->bytes && job->after_last_copy && job->after_last_copy(*job) != 0)
        return fail("completion event of a staged evict failed");
    }
    // 4. jobs whose every chunk is in the file
    for (StagedJob* job : jobs_)
      if (!job->finished && job->written.load(std::memory_order_acquire) == job->bytes) {
        job->finished = true;
        if (job->on_durable) job->on_durable(*job);
        ++moved;
      }
  }
  while (!jobs_.empty() && jobs_.front()->finished) {
    jobs_.pop_front();
    if (read_cursor_ > 0) --read_cursor_;
    ++moved;
  }
  return moved;
}

}  // namespace ssc
