// Submitter thread of the batch feeder in native code: packs the batches of one pass over a packed
// data set into a ring of pinned host arenas and uploads each with one asynchronous copy on its own
// copy stream, ahead of the consumer.  The reference does this with a Python thread that runs
// feed_dict into a TensorFlow FIFOQueue (khan/training/trainer_multi_tower.py:749-828); a Python
// submitter shares the interpreter lock with the consumer's per-batch work and was what bounded
// predict / coordinate_gradients / feed_dataset once the kernels were fast.  Here the consumer's
// only call per batch (next) blocks outside the interpreter lock.
//
// Ordering, all on the device except where said:
//   - the copy of batch b into a slot's device arena waits (cudaStreamWaitEvent on the copy stream)
//     for the event the consumer recorded when it released the slot's previous batch;
//   - the pinned host arena is rewritten only after the slot's previous copy has finished (the
//     submitter thread waits for that event on the host);
//   - the consumer's stream waits for the slot's "uploaded" event (wait()).
// With device < 0 nothing is copied and no CUDA call is made: the consumer reads the host arenas.
#pragma once

#include <condition_variable>
#include <cstdint>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/ani_b200.h"
#include "ani_host_pack.h"

namespace ani {

struct FeederSlot {
    ani_host_pack_args args{};   // source and destination pointers of this slot; picks are set per batch
    void* host_arena = nullptr;
    void* dev_arena = nullptr;
    size_t nbytes = 0;
    cudaEvent_t uploaded = nullptr, consumed = nullptr;
    bool has_uploaded = false, has_consumed = false;
    int n_atoms = 0, n_mols = 0, acs[4] = {0, 0, 0, 0};
    long long batch_index = -1;
};

class Feeder {
public:
    Feeder(int device, const ani_feeder_slot* slots, int n_slots) : device_(device), slots_(n_slots)
    {
        for (int s = 0; s < n_slots; s++) {
            slots_[s].args = slots[s].pack;
            slots_[s].host_arena = slots[s].host_arena;
            slots_[s].dev_arena = slots[s].dev_arena;
            slots_[s].nbytes = slots[s].nbytes;
        }
    }

    int init()
    {
        if (device_ < 0) return ANI_OK;
        int prev = 0;
        if (cudaGetDevice(&prev) != cudaSuccess || cudaSetDevice(device_) != cudaSuccess) return ANI_ERR_CUDA;
        int rc = ANI_OK;
        if (cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking) != cudaSuccess) rc = ANI_ERR_CUDA;
        for (auto& s : slots_) {
            if (rc) break;
            if (cudaEventCreateWithFlags(&s.uploaded, cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&s.consumed, cudaEventDisableTiming) != cudaSuccess)
                rc = ANI_ERR_CUDA;
        }
        cudaSetDevice(prev);
        return rc;
    }

    ~Feeder()
    {
        end();
        for (auto& s : slots_) {
            if (s.uploaded) cudaEventDestroy(s.uploaded);
            if (s.consumed) cudaEventDestroy(s.consumed);
        }
        if (copy_stream_) cudaStreamDestroy(copy_stream_);
    }

    // Starts a pass: batch b is the molecules order[b * batch_size ... ) of the data set.
    int begin(const long long* order, long long n_order, int batch_size)
    {
        if (n_order < 0 || batch_size <= 0 || (n_order > 0 && !order)) return ANI_ERR_BAD_SIZE;
        end();
        order_.assign(order, order + n_order);
        batch_size_ = batch_size;
        n_batches_ = (n_order + batch_size - 1) / batch_size;
        {
            std::lock_guard<std::mutex> lk(mu_);
            stop_ = false;
            finished_ = false;
            error_ = ANI_OK;
            free_.clear();
            ready_.clear();
            for (int s = 0; s < (int)slots_.size(); s++) free_.push_back(s);
        }
        thread_ = std::thread([this] { run(); });
        return ANI_OK;
    }

    // Blocks until the next batch has been packed and its copy enqueued.  1: *out is a batch;
    // 0: the pass is over; negative: the submitter failed with that code.
    int next(ani_feeder_batch* out)
    {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [this] { return !ready_.empty() || finished_ || stop_; });
        if (ready_.empty()) return error_ ? error_ : 0;
        const int s = ready_.front();
        ready_.pop_front();
        const FeederSlot& sl = slots_[s];
        out->slot = s;
        out->batch_index = sl.batch_index;
        out->n_atoms = sl.n_atoms;
        out->n_mols = sl.n_mols;
        for (int t = 0; t < 4; t++) out->acs[t] = sl.acs[t];
        return 1;
    }

    // The consumer's stream waits for the upload of the batch in `slot`.
    int wait(int slot, cudaStream_t stream)
    {
        if (slot < 0 || slot >= (int)slots_.size()) return ANI_ERR_BAD_INDEX;
        if (device_ < 0 || !slots_[slot].has_uploaded) return ANI_OK;
        return cudaStreamWaitEvent(stream, slots_[slot].uploaded, 0) == cudaSuccess ? ANI_OK : ANI_ERR_CUDA;
    }

    // Hands the slot back: the next copy into its device arena is ordered behind the work enqueued on
    // `stream` so far.
    int release(int slot, cudaStream_t stream)
    {
        if (slot < 0 || slot >= (int)slots_.size()) return ANI_ERR_BAD_INDEX;
        if (device_ >= 0) {
            if (cudaEventRecord(slots_[slot].consumed, stream) != cudaSuccess) return ANI_ERR_CUDA;
        }
        {
            std::lock_guard<std::mutex> lk(mu_);
            slots_[slot].has_consumed = device_ >= 0;
            free_.push_back(slot);
        }
        cv_.notify_all();
        return ANI_OK;
    }

    // Stops the submitter (if a pass is running) and waits for it.  Copies already enqueued finish on
    // their own; the arenas must stay alive until then (the owner synchronises before freeing them).
    void end()
    {
        {
            std::lock_guard<std::mutex> lk(mu_);
            stop_ = true;
        }
        cv_.notify_all();
        if (thread_.joinable()) thread_.join();
    }

    // Host wait for every copy this feeder has enqueued (before the arenas are reused elsewhere).
    int drain()
    {
        if (device_ < 0 || !copy_stream_) return ANI_OK;
        return cudaStreamSynchronize(copy_stream_) == cudaSuccess ? ANI_OK : ANI_ERR_CUDA;
    }

private:
    void fail(int code)
    {
        {
            std::lock_guard<std::mutex> lk(mu_);
            error_ = code;
            finished_ = true;
        }
        cv_.notify_all();
    }

    void run()
    {
        if (device_ >= 0 && cudaSetDevice(device_) != cudaSuccess) return fail(ANI_ERR_CUDA);
        const long long n_order = (long long)order_.size();
        for (long long b = 0; b < n_batches_; b++) {
            int s;
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [this] { return !free_.empty() || stop_; });
                if (stop_) return;
                s = free_.front();
                free_.pop_front();
            }
            FeederSlot& sl = slots_[s];
            if (sl.has_uploaded) {   // the pinned arena is still the source of this slot's previous copy
                if (cudaEventSynchronize(sl.uploaded) != cudaSuccess) return fail(ANI_ERR_CUDA);
                sl.has_uploaded = false;
            }
            const long long first = b * batch_size_;
            ani_host_pack_args a = sl.args;
            a.picks = order_.data() + first;
            a.n_picks = (int)((n_order - first < batch_size_) ? n_order - first : batch_size_);
            a.noise = nullptr;
            a.n_atoms_out = &sl.n_atoms;
            a.acs_out = sl.acs;
            if (int rc = host_pack_batch(a)) return fail(rc);
            sl.n_mols = a.n_picks;
            sl.batch_index = b;
            if (device_ >= 0) {
                if (sl.has_consumed && cudaStreamWaitEvent(copy_stream_, sl.consumed, 0) != cudaSuccess)
                    return fail(ANI_ERR_CUDA);
                sl.has_consumed = false;
                if (cudaMemcpyAsync(sl.dev_arena, sl.host_arena, sl.nbytes, cudaMemcpyHostToDevice, copy_stream_) !=
                        cudaSuccess ||
                    cudaEventRecord(sl.uploaded, copy_stream_) != cudaSuccess)
                    return fail(ANI_ERR_CUDA);
                sl.has_uploaded = true;
            }
            {
                std::lock_guard<std::mutex> lk(mu_);
                ready_.push_back(s);
            }
            cv_.notify_all();
        }
        {
            std::lock_guard<std::mutex> lk(mu_);
            finished_ = true;
        }
        cv_.notify_all();
    }

    int device_;
    cudaStream_t copy_stream_ = nullptr;
    std::vector<FeederSlot> slots_;
    std::vector<long long> order_;
    int batch_size_ = 1;
    long long n_batches_ = 0;
    std::thread thread_;
    std::mutex mu_;
    std::condition_variable cv_;
    std::deque<int> free_, ready_;
    bool stop_ = true, finished_ = true;
    int error_ = ANI_OK;
};

}  // namespace ani
