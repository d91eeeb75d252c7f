// Column-sharded int8 Linear across the GPUs of one node, host side in C++ over the C ABI
// (include/nnb200.h): one process per GPU, rank r owns output channels [r*N/g, (r+1)*N/g) and
// the matching rows of W [N, K]; the GEMM's epilogue stores every finished tile into every
// rank's copy of the full [M, N] output (peer-to-peer stores into CUDA-IPC-mapped buffers), and
// a device-side flag barrier orders the ranks.  Each output element is produced by exactly one
// GPU from the same integer inputs, so the g-way result is byte-identical to the single-GPU one.
//
// The reference has no multi-GPU code; this sits above its operator API, one instance per GPU.
//
// What the ranks have to tell each other on the host -- 64-byte IPC handles once, "still there?"
// before a step -- goes through a ShardExchange, an interface any launcher can implement (MPI, a
// TCP store, ...).  LocalExchange is one for processes of one machine over POSIX shared memory;
// it is also where a lost rank is noticed WITHOUT touching a GPU: a rank that announces its
// leaving makes the others' next exchange fail at once, one that dies silently or never joins
// makes it fail at the deadline.  Header-only, C++17, no CUDA headers.
#pragma once

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "nnb200.h"

namespace nnops::b200 {

constexpr int kMaxShardRanks = 8;   // nnb200_rank_barrier's limit: one NVSwitch domain

// Fixed-size all-gather and barrier among the ranks, with a deadline.
class ShardExchange {
public:
    virtual ~ShardExchange() = default;
    virtual int rank() const = 0;
    virtual int world() const = 0;
    // Every rank contributes `bytes` (<= max_bytes()); `all` receives world() * bytes in rank
    // order.  false: a rank has left or was not heard from in time (lost_rank() names it).
    virtual bool all_gather(const void* mine, void* all, size_t bytes) = 0;
    virtual size_t max_bytes() const = 0;
    virtual int lost_rank() const = 0;
    bool barrier()
    {
        uint8_t mine = 1, all[kMaxShardRanks];
        return all_gather(&mine, all, 1);
    }
};

// ShardExchange for the processes of one machine: a POSIX shared-memory segment `name`, created
// by whichever rank arrives first.  Step s of the exchange: write the payload into slot
// [s & 1][rank], publish seq[rank] = s + 1, wait until every seq[r] >= s + 1, copy everything
// out.  Two slots suffice: a rank reaches step s + 2 (which reuses slot s & 1) only after every
// rank has published step s + 1, i.e. has finished reading step s.
class LocalExchange final : public ShardExchange {
public:
    static constexpr size_t kSlotBytes = 1024;

    LocalExchange(const std::string& name, int rank, int world, double timeout_s = 30.0)
        : name_(name), rank_(rank), world_(world), timeout_s_(timeout_s)
    {
        if (world < 1 || world > kMaxShardRanks || rank < 0 || rank >= world) {
            return;
        }
        const int fd = shm_open(name.c_str(), O_CREAT | O_RDWR, 0600);
        if (fd < 0) {
            return;
        }
        if (ftruncate(fd, sizeof(Segment)) != 0) {   // new pages read as zero: every counter starts at 0
            ::close(fd);
            return;
        }
        void* p = mmap(nullptr, sizeof(Segment), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
        ::close(fd);
        if (p == MAP_FAILED) {
            return;
        }
        seg_ = static_cast<Segment*>(p);
    }
    ~LocalExchange() override
    {
        if (seg_ != nullptr) {
            munmap(seg_, sizeof(Segment));
        }
    }
    LocalExchange(const LocalExchange&) = delete;
    LocalExchange& operator=(const LocalExchange&) = delete;

    bool ok() const { return seg_ != nullptr; }
    int rank() const override { return rank_; }
    int world() const override { return world_; }
    size_t max_bytes() const override { return kSlotBytes; }
    int lost_rank() const override { return lost_; }
    void set_timeout(double seconds) { timeout_s_ = seconds; }

    // Announce that this rank is going: the others' exchanges fail at once instead of at the
    // deadline.  Call it between steps, with none of this rank's kernels in flight.
    void leave()
    {
        if (seg_ != nullptr) {
            seg_->left[rank_].store(1, std::memory_order_release);
        }
    }
    // Remove the segment's name (any one rank, after the last exchange).
    void unlink() { shm_unlink(name_.c_str()); }

    bool all_gather(const void* mine, void* all, size_t bytes) override
    {
        if (seg_ == nullptr || bytes > kSlotBytes || lost_ >= 0) {
            return false;
        }
        const uint32_t s = step_;
        std::memcpy(seg_->slot[s & 1u][rank_], mine, bytes);
        seg_->seq[rank_].store(s + 1, std::memory_order_release);
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(timeout_s_);
        for (int r = 0; r < world_; ++r) {
            unsigned spins = 0;
            // seq counts up and never wraps in a job's life; signed difference all the same.
            while (static_cast<int32_t>(seg_->seq[r].load(std::memory_order_acquire) - (s + 1)) < 0) {
                if (seg_->left[r].load(std::memory_order_acquire) != 0 || std::chrono::steady_clock::now() > deadline) {
                    lost_ = r;
                    return false;
                }
                if (++spins > 64) {
                    std::this_thread::sleep_for(std::chrono::microseconds(50));
                }
            }
        }
        for (int r = 0; r < world_; ++r) {
            std::memcpy(static_cast<uint8_t*>(all) + static_cast<size_t>(r) * bytes, seg_->slot[s & 1u][r], bytes);
        }
        ++step_;
        return true;
    }

private:
    struct Segment {
        std::atomic<uint32_t> seq[kMaxShardRanks];
        std::atomic<uint32_t> left[kMaxShardRanks];
        uint8_t slot[2][kMaxShardRanks][kSlotBytes];
    };
    static_assert(std::atomic<uint32_t>::is_always_lock_free, "shared-memory counters must be lock-free");

    std::string name_;
    int rank_, world_;
    double timeout_s_;
    Segment* seg_ = nullptr;
    uint32_t step_ = 0;
    int lost_ = -1;
};

// The layer.  `shard` describes THIS rank's GEMM exactly as a single-GPU call would: w, bias,
// scale_w, zp_w are the rank's own rows / entries, n = N / g, out_kind S8 or U8, everything
// else as for nnb200_gemm_i8; a, out, ldc, m and the peer fields are filled in per call.
// Every method returns an NNB200_* status; all ranks must make the same calls in the same order.
class ShardedLinearI8 {
public:
    ShardedLinearI8(ShardExchange& exchange, const nnb200_gemm_i8_args& shard, int64_t n_total)
        : ex_(exchange), shard_(shard), n_total_(n_total)
    {
    }
    ~ShardedLinearI8() { release(); }
    ShardedLinearI8(const ShardedLinearI8&) = delete;
    ShardedLinearI8& operator=(const ShardedLinearI8&) = delete;

    int64_t col0() const { return static_cast<int64_t>(ex_.rank()) * shard_.n; }
    int lost_rank() const { return ex_.lost_rank(); }

    // `count` full [m, n_total] 8-bit outputs on this rank, every one of them mapped by every
    // other rank, plus the flag arrays of the device-side barrier.  The device that will run
    // the kernels must be current.
    int alloc_outputs(int64_t m, int count)
    {
        const int g = ex_.world(), me = ex_.rank();
        if (!outs_.empty() || flag_.own != nullptr) {
            return NNB200_INVALID_ARGUMENT;   // one allocation per layer: close() first
        }
        if (g < 1 || g > kMaxShardRanks || count < 1 || m < 1 || shard_.n * g != n_total_ ||
            (shard_.out_kind != NNB200_OUT_S8 && shard_.out_kind != NNB200_OUT_U8)) {
            return NNB200_INVALID_ARGUMENT;
        }
        m_ = m;
        std::vector<uint8_t> everyone(static_cast<size_t>(g) * 64);
        for (int i = 0; i <= count; ++i) {   // i == count: the flag array
            const bool flags = i == count;
            if (flags && g == 1) {
                break;
            }
            if (!flags) {
                outs_.emplace_back();
            }
            Buffer& slot = flags ? flag_ : outs_.back();   // owned from here on: release() frees it on any exit
            slot.mapped.assign(static_cast<size_t>(g), nullptr);
            const size_t bytes = flags ? NNB200_RANK_FLAG_BYTES : static_cast<size_t>(m) * static_cast<size_t>(n_total_);
            int st = nnb200_peer_buffer_alloc(&slot.own, bytes);
            if (st != NNB200_OK) {
                return st;
            }
            slot.mapped[static_cast<size_t>(me)] = slot.own;
            if (flags) {
                // Zeroed once, before anyone can write into it: the exchange below orders that.
                std::vector<uint8_t> zero(NNB200_RANK_FLAG_BYTES, 0);
                st = nnb200_copy_h2d_async(slot.own, zero.data(), zero.size(), nullptr);
                int32_t code = 0;
                if (st != NNB200_OK || (st = nnb200_take_device_error(&code)) != NNB200_OK) {
                    return st;
                }
            }
            if (g == 1) {
                continue;
            }
            uint8_t handle[64];
            st = nnb200_peer_buffer_export(slot.own, handle);
            if (st != NNB200_OK) {
                return st;
            }
            if (!ex_.all_gather(handle, everyone.data(), 64)) {
                return NNB200_INTERNAL;
            }
            for (int r = 0; r < g; ++r) {
                if (r != me) {
                    st = nnb200_peer_buffer_open(everyone.data() + static_cast<size_t>(r) * 64, &slot.mapped[static_cast<size_t>(r)]);
                    if (st != NNB200_OK) {
                        return st;
                    }
                }
            }
        }
        // Every rank has mapped everything before anyone launches.
        return (g == 1 || ex_.barrier()) ? NNB200_OK : NNB200_INTERNAL;
    }

    void* output(int i) const { return outs_[static_cast<size_t>(i)].own; }

    // Host-side check, before anything is launched, that every rank is still there.
    int begin_step() { return (ex_.world() == 1 || ex_.barrier()) ? NNB200_OK : NNB200_INTERNAL; }

    // out[i] = epilogue(A [m, k] x W^T) on every rank.  wait_for_readers: order the ranks BEFORE
    // the GEMM as well, for callers whose previous result in that buffer may still be read on
    // another rank.  Work enqueued on `stream` afterwards sees the whole output.
    int forward(const void* a, int64_t lda, int out_index, void* stream, bool wait_for_readers = false)
    {
        if (out_index < 0 || out_index >= static_cast<int>(outs_.size())) {
            return NNB200_INVALID_ARGUMENT;
        }
        const int g = ex_.world(), me = ex_.rank();
        const Buffer& o = outs_[static_cast<size_t>(out_index)];
        if (wait_for_readers && g > 1) {
            const int st = rank_barrier(stream);
            if (st != NNB200_OK) {
                return st;
            }
        }
        nnb200_gemm_i8_args c = shard_;
        c.a = a;
        c.a_stride_m = lda;
        c.a_stride_k = 1;
        c.m = m_;
        c.batch = 1;
        c.ldc = n_total_;
        c.out = static_cast<uint8_t*>(o.own) + col0();
        c.num_peer_outs = 0;
        for (int r = 0; r < g; ++r) {
            if (r != me) {
                c.peer_out[c.num_peer_outs++] = static_cast<uint8_t*>(o.mapped[static_cast<size_t>(r)]) + col0();
            }
        }
        const int st = nnb200_gemm_i8(&c, stream);
        if (st != NNB200_OK || g == 1) {
            return st;
        }
        return rank_barrier(stream);   // every rank's tiles have landed in every copy
    }

    // Synchronise this rank's device and report whether a bounded wait ran out since the last
    // check: the outputs gathered since then are valid only if this returns NNB200_OK.
    int check()
    {
        int32_t code = 0;
        const int st = nnb200_take_device_error(&code);
        return st != NNB200_OK ? st : (code == 0 ? NNB200_OK : NNB200_INTERNAL);
    }

    // Unmap and free while every rank is still alive: the ranks meet, each drops its mappings,
    // they meet again, each frees its own buffers.  NNB200_INTERNAL if a rank was lost on the
    // way (the buffers are released all the same).
    int close()
    {
        bool met = true;
        if (ex_.world() > 1) {
            int32_t code = 0;
            nnb200_take_device_error(&code);   // synchronises the device
            met = ex_.barrier();
        }
        unmap();
        if (ex_.world() > 1 && met) {
            met = ex_.barrier();
        }
        release();
        return met ? NNB200_OK : NNB200_INTERNAL;
    }

private:
    struct Buffer {
        void* own = nullptr;
        std::vector<void*> mapped;   // by rank; [rank()] == own
    };

    int rank_barrier(void* stream)
    {
        int32_t* table[kMaxShardRanks] = {};
        for (int r = 0; r < ex_.world(); ++r) {
            table[r] = static_cast<int32_t*>(flag_.mapped[static_cast<size_t>(r)]);
        }
        return nnb200_rank_barrier(table, ex_.world(), ex_.rank(), 0, stream);
    }
    void unmap()
    {
        const auto drop = [&](Buffer& b) {
            for (size_t r = 0; r < b.mapped.size(); ++r) {
                if (b.mapped[r] != nullptr && b.mapped[r] != b.own) {
                    nnb200_peer_buffer_close(b.mapped[r]);
                }
                b.mapped[r] = nullptr;
            }
        };
        for (Buffer& b : outs_) {
            drop(b);
        }
        drop(flag_);
    }
    void release()
    {
        unmap();
        for (Buffer& b : outs_) {
            if (b.own != nullptr) {
                nnb200_peer_buffer_free(b.own);
            }
        }
        outs_.clear();
        if (flag_.own != nullptr) {
            nnb200_peer_buffer_free(flag_.own);
            flag_.own = nullptr;
        }
    }

    ShardExchange& ex_;
    nnb200_gemm_i8_args shard_;
    int64_t n_total_;
    int64_t m_ = 0;
    std::vector<Buffer> outs_;
    Buffer flag_;
};

}  // namespace nnops::b200
