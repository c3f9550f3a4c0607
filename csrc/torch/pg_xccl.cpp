// PyTorch c10d backend over the xccl C API ("b200xccl").
//
// The reference ships an Open MPI coll component as its framework binding
// (ompi_coll_xccl.patch: lazy lib/context creation, one team per communicator, an OOB allgather
// built on the host framework's own messaging, fallback on unsupported calls). This is the same
// role for torch.distributed: one xccl team per process group, the OOB allgather built on the
// c10d Store, CUDA collectives enqueued on a dedicated high-priority stream and completed
// through CUDA-aware futures so DistributedDataParallel overlaps them with backward.
// An extra entry point, allreduce_fused, exposes the scale + cast epilogue for gradient buckets.
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <ATen/cuda/CUDAEvent.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <torch/python.h>
#include <pybind11/chrono.h>

#include <chrono>
#include <cstdlib>
#include <map>
#include <memory>
#include <sstream>

#include "xccl/xccl.h"
#include "xccl/xccl_oob.h"
#include "../tl/nccl/nccl_tl.h"  // xccl_p2p_* (extension: point-to-point on NCCL)

namespace {

void check(xccl_status_t st, const char *what)
{
    TORCH_CHECK(st == XCCL_OK, "xccl: ", what, " failed: ", xccl_status_str(st));
}

xccl_dt_t to_dt(at::ScalarType t)
{
    switch (t) {
    case at::kChar: return XCCL_DT_INT8;
    case at::kByte: return XCCL_DT_UINT8;
    case at::kBool: return XCCL_DT_UINT8;
    case at::kShort: return XCCL_DT_INT16;
    case at::kInt: return XCCL_DT_INT32;
    case at::kLong: return XCCL_DT_INT64;
    case at::kHalf: return XCCL_DT_FLOAT16;
    case at::kBFloat16: return XCCL_DT_BFLOAT16;
    case at::kFloat: return XCCL_DT_FLOAT32;
    case at::kDouble: return XCCL_DT_FLOAT64;
    default: TORCH_CHECK(false, "xccl: unsupported tensor dtype ", t);
    }
}

xccl_op_t to_op(const c10d::ReduceOp &op)
{
    switch (op.op_) {
    case c10d::ReduceOp::SUM:
    case c10d::ReduceOp::AVG: return XCCL_OP_SUM;
    case c10d::ReduceOp::PRODUCT: return XCCL_OP_PROD;
    case c10d::ReduceOp::MIN: return XCCL_OP_MIN;
    case c10d::ReduceOp::MAX: return XCCL_OP_MAX;
    case c10d::ReduceOp::BAND: return XCCL_OP_BAND;
    case c10d::ReduceOp::BOR: return XCCL_OP_BOR;
    case c10d::ReduceOp::BXOR: return XCCL_OP_BXOR;
    default: TORCH_CHECK(false, "xccl: unsupported reduce op");
    }
}

// ------------------------------------------------------------------ OOB over the c10d store
struct StoreOob {
    c10::intrusive_ptr<c10d::Store> store;
    int                             rank, size;
    std::map<std::string, uint64_t> counters;  // per member-set sequence numbers
    std::string                     prefix;    // key namespace (pairwise bootstraps of send/recv use their own)
};

struct StoreReq {
    StoreOob                *oob;
    std::vector<std::string> keys;
    char                    *rbuf;
    size_t                   bytes;
};

int store_allgather(void *sbuf, void *rbuf, size_t bytes, int my_rank, xccl_ep_range_t range, void *ctx, void **request)
{
    auto            *o = static_cast<StoreOob *>(ctx);
    std::vector<int> members;
    if (range.type == XCCL_EP_RANGE_UNDEFINED) {
        for (int i = 0; i < o->size; i++) members.push_back(i);
        my_rank = o->rank;
    } else {
        for (int i = 0; i < range.ep_num; i++) members.push_back(xccl_range_to_rank(range, i));
    }
    std::ostringstream sig;
    for (int m : members) sig << m << ".";
    uint64_t    seq  = o->counters[sig.str()]++;
    std::string base = "xccl/oob/" + o->prefix + sig.str() + "/" + std::to_string(seq) + "/";
    auto       *r    = new StoreReq{o, {}, static_cast<char *>(rbuf), bytes};
    for (size_t i = 0; i < members.size(); i++) r->keys.push_back(base + std::to_string(i));
    std::vector<uint8_t> mine(static_cast<uint8_t *>(sbuf), static_cast<uint8_t *>(sbuf) + bytes);
    if (mine.empty()) mine.push_back(0);
    o->store->set(r->keys[static_cast<size_t>(my_rank)], mine);
    *request = r;
    return 0;
}

xccl_status_t store_test(void *request)
{
    auto *r = static_cast<StoreReq *>(request);
    if (!r->oob->store->check(r->keys)) return XCCL_INPROGRESS;
    for (size_t i = 0; i < r->keys.size(); i++) {
        std::vector<uint8_t> v = r->oob->store->get(r->keys[i]);
        if (r->bytes > 0) std::memcpy(r->rbuf + i * r->bytes, v.data(), std::min(r->bytes, v.size()));
    }
    return XCCL_OK;
}

xccl_status_t store_free(void *request)
{
    delete static_cast<StoreReq *>(request);
    return XCCL_OK;
}

// ------------------------------------------------------------------ work
class WorkXccl : public c10d::Work {
public:
    WorkXccl(c10d::OpType op, std::vector<at::Tensor> outputs, bool cuda)
        : c10d::Work(-1, op), outputs_(std::move(outputs))
    {
        std::vector<c10::Device> devs;
        if (cuda && !outputs_.empty()) devs.push_back(outputs_[0].device());
        future_ = c10::make_intrusive<at::ivalue::Future>(c10::ListType::create(c10::TensorType::get()), devs);
    }
    // called with the communication stream current: the future records its events on it
    void complete() { future_->markCompleted(at::IValue(outputs_)); }
    bool isCompleted() override { return future_->completed(); }
    bool isSuccess() const override { return future_->hasValue(); }
    bool wait(std::chrono::milliseconds) override
    {
        future_->wait();  // for CUDA: makes the current stream wait, does not block the host
        return true;
    }
    c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }
    std::vector<at::Tensor>                 result() override { return outputs_; }

private:
    std::vector<at::Tensor>                 outputs_;
    c10::intrusive_ptr<c10::ivalue::Future> future_;
};

// ------------------------------------------------------------------ backend
class ProcessGroupXccl : public c10d::Backend {
public:
    ProcessGroupXccl(const c10::intrusive_ptr<c10d::Store> &store, int rank, int size) : c10d::Backend(rank, size)
    {
        oob_state_ = StoreOob{store, rank, size, {}, ""};
        oob_.allgather    = store_allgather;
        oob_.req_test     = store_test;
        oob_.req_free     = store_free;
        oob_.coll_context = &oob_state_;
        oob_.rank         = rank;
        oob_.size         = size;
        xccl_lib_params_t lp{};
        check(xccl_lib_init(&lp, nullptr, &lib_), "xccl_lib_init");
        const char *tls_env = std::getenv("XCCL_TORCH_TLS");
        uint64_t    tls     = xccl_tls_str_to_bitmap(tls_env != nullptr ? tls_env : "nvlink,nccl,ucx");
        xccl_context_params_t cp{};
        cp.field_mask  = XCCL_CONTEXT_PARAM_FIELD_OOB | XCCL_CONTEXT_PARAM_FIELD_TLS | XCCL_CONTEXT_PARAM_FIELD_THREAD_MODE;
        cp.thread_mode = XCCL_THREAD_MODE_SINGLE;
        cp.oob         = oob_;
        cp.tls         = tls;
        check(xccl_context_create(lib_, &cp, nullptr, &ctx_), "xccl_context_create");
        xccl_team_params_t tp{};
        tp.field_mask   = XCCL_TEAM_PARAM_FIELD_EP_RANGE;
        tp.range.type   = XCCL_EP_RANGE_FULL;
        tp.range.ep_num = size;
        check(xccl_team_create_post(ctx_, &tp, &team_), "xccl_team_create_post");
        xccl_status_t st;
        while ((st = xccl_team_create_test(team_)) == XCCL_INPROGRESS) xccl_context_progress(ctx_);
        check(st, "xccl_team_create_test");
    }

    ~ProcessGroupXccl() override
    {
        for (auto &kv : pairs_) xccl_p2p_comm_destroy(kv.second->comm);
        if (team_ != nullptr) xccl_team_destroy(team_);
        if (ctx_ != nullptr) xccl_context_destroy(ctx_);
        if (lib_ != nullptr) xccl_lib_cleanup(lib_);
    }

    const std::string getBackendName() const override { return "b200xccl"; }

    // True when the team library that serves `coll` on device memory enqueues all of its work on the stream
    // it is given, so that a later event on that stream stands for completion.
    bool stream_ordered(xccl_collective_type_t coll) const
    {
        xccl_tl_id_t id = xccl_team_coll_tl(team_, coll, XCCL_MEMORY_TYPE_CUDA);
        return id == XCCL_TL_NVLINK || id == XCCL_TL_NCCL || id == XCCL_TL_SHARP || id == XCCL_TL_HMC;
    }

    // A tensor in symmetric memory of the team (xccl_team_mem_alloc; collective: every rank calls it with the same
    // size). Collectives on such tensors, at the same offset on every rank, run zero-copy through the NVSwitch
    // multicast mapping. The memory is returned when the last reference to the tensor goes - call
    // free_symmetric (collective) explicitly where the ranks must agree on the moment.
    at::Tensor empty_symmetric(int64_t nbytes, c10::DeviceIndex dev)
    {
        c10::cuda::CUDAGuard guard(dev);
        void *p = nullptr;
        check(xccl_team_mem_alloc(team_, static_cast<size_t>(nbytes), &p), "xccl_team_mem_alloc");
        return at::from_blob(p, {nbytes}, [](void *) {}, at::TensorOptions().dtype(at::kByte).device(at::kCUDA, dev));
    }
    void free_symmetric(const at::Tensor &t) { check(xccl_team_mem_free(team_, t.data_ptr()), "xccl_team_mem_free"); }

    // Which team library serves a collective for a memory type (for tests and logs).
    std::string coll_tl(int coll, bool cuda) const
    {
        xccl_tl_id_t id = xccl_team_coll_tl(team_, static_cast<xccl_collective_type_t>(coll),
                                            cuda ? XCCL_MEMORY_TYPE_CUDA : XCCL_MEMORY_TYPE_HOST);
        const char  *n  = xccl_tl_str(id);
        return n != nullptr ? n : "none";
    }

    c10::intrusive_ptr<c10d::Work> run(xccl_coll_op_args_t &args, c10d::OpType op, std::vector<at::Tensor> outputs,
                                       const std::vector<at::Tensor> &touched)
    {
        bool cuda = !touched.empty() && touched[0].is_cuda();
        auto work = c10::make_intrusive<WorkXccl>(op, std::move(outputs), cuda);
        if (cuda) {
            c10::cuda::CUDAGuard dev_guard(touched[0].device());
            auto                 cur  = c10::cuda::getCurrentCUDAStream();
            auto                 comm = comm_stream(touched[0].device().index());
            at::cuda::CUDAEvent  ready;
            ready.record(cur);
            ready.block(comm);
            for (const auto &t : touched) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), comm);
            cudaStream_t raw   = comm.stream();
            args.field_mask   |= XCCL_COLL_OP_ARGS_FIELD_STREAM;
            args.stream.type   = XCCL_STREAM_TYPE_CUDA;
            args.stream.stream = &raw;
            xccl_coll_req_h req = nullptr;
            check(xccl_collective_init(&args, &req, team_), "xccl_collective_init");
            check(xccl_collective_post(req), "xccl_collective_post");
            if (stream_ordered(args.coll_type)) {
                pending_.push_back(req);
                reap(false);
            } else {
                // a host-progressed team library (the host team staging device buffers, or a composite one):
                // its result is complete only when test says so, nothing on the stream stands for it
                check(xccl_collective_wait(req), "xccl_collective_wait");
                check(xccl_collective_finalize(req), "xccl_collective_finalize");
            }
            c10::cuda::CUDAStreamGuard guard(comm);
            work->complete();
        } else {
            xccl_coll_req_h req = nullptr;
            check(xccl_collective_init(&args, &req, team_), "xccl_collective_init");
            check(xccl_collective_post(req), "xccl_collective_post");
            check(xccl_collective_wait(req), "xccl_collective_wait");
            check(xccl_collective_finalize(req), "xccl_collective_finalize");
            work->complete();
        }
        return work;
    }

    c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor> &tensors, const c10d::AllreduceOptions &opts) override
    {
        TORCH_CHECK(tensors.size() == 1, "xccl: one tensor per allreduce");
        at::Tensor &t = tensors[0];
        TORCH_CHECK(t.is_contiguous(), "xccl: tensor must be contiguous");
        xccl_coll_op_args_t a{};
        a.coll_type              = XCCL_ALLREDUCE;
        a.buffer_info.src_buffer = t.data_ptr();
        a.buffer_info.dst_buffer = t.data_ptr();
        a.buffer_info.len        = t.nbytes();
        a.reduce_info.dt         = to_dt(t.scalar_type());
        a.reduce_info.op         = to_op(opts.reduceOp);
        a.reduce_info.count      = static_cast<size_t>(t.numel());
        if (opts.reduceOp.op_ == c10d::ReduceOp::AVG) {
            a.field_mask |= XCCL_COLL_OP_ARGS_FIELD_EPILOGUE;
            a.epilogue.scale  = 1.0f / static_cast<float>(getSize());
            a.epilogue.out_dt = XCCL_DT_UNSUPPORTED;
        }
        return run(a, c10d::OpType::ALLREDUCE, tensors, tensors);
    }

    // out = cast(scale * sum over ranks of in): the gradient-bucket form (no separate div / cast pass)
    c10::intrusive_ptr<c10d::Work> allreduce_fused(at::Tensor in, at::Tensor out, double scale)
    {
        TORCH_CHECK(in.is_contiguous() && out.is_contiguous() && in.numel() == out.numel(), "xccl: bad fused allreduce tensors");
        xccl_coll_op_args_t a{};
        a.coll_type              = XCCL_ALLREDUCE;
        a.field_mask             = XCCL_COLL_OP_ARGS_FIELD_EPILOGUE;
        a.buffer_info.src_buffer = in.data_ptr();
        a.buffer_info.dst_buffer = out.data_ptr();
        a.buffer_info.len        = in.nbytes();
        a.reduce_info.dt         = to_dt(in.scalar_type());
        a.reduce_info.op         = XCCL_OP_SUM;
        a.reduce_info.count      = static_cast<size_t>(in.numel());
        a.epilogue.scale         = static_cast<float>(scale);
        a.epilogue.out_dt        = to_dt(out.scalar_type());
        return run(a, c10d::OpType::ALLREDUCE, {out}, {in, out});
    }

    c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor> &tensors, const c10d::BroadcastOptions &opts) override
    {
        TORCH_CHECK(tensors.size() == 1 && tensors[0].is_contiguous(), "xccl: one contiguous tensor per broadcast");
        at::Tensor         &t = tensors[0];
        xccl_coll_op_args_t a{};
        a.coll_type              = XCCL_BCAST;
        a.buffer_info.src_buffer = t.data_ptr();
        a.buffer_info.dst_buffer = t.data_ptr();
        a.buffer_info.len        = t.nbytes();
        a.root                   = static_cast<int>(opts.rootRank);
        return run(a, c10d::OpType::BROADCAST, tensors, tensors);
    }

    c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor> &tensors, const c10d::ReduceOptions &opts) override
    {
        TORCH_CHECK(tensors.size() == 1 && tensors[0].is_contiguous(), "xccl: one contiguous tensor per reduce");
        at::Tensor         &t = tensors[0];
        xccl_coll_op_args_t a{};
        a.coll_type              = XCCL_REDUCE;
        a.buffer_info.src_buffer = t.data_ptr();
        a.buffer_info.dst_buffer = t.data_ptr();
        a.buffer_info.len        = t.nbytes();
        a.reduce_info.dt         = to_dt(t.scalar_type());
        a.reduce_info.op         = to_op(opts.reduceOp);
        a.reduce_info.count      = static_cast<size_t>(t.numel());
        a.root                   = static_cast<int>(opts.rootRank);
        return run(a, c10d::OpType::REDUCE, tensors, tensors);
    }

    c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor &out, at::Tensor &in, const c10d::AllgatherOptions &) override
    {
        TORCH_CHECK(out.is_contiguous() && in.is_contiguous() && out.nbytes() == in.nbytes() * static_cast<size_t>(getSize()),
                    "xccl: bad allgather tensors");
        xccl_coll_op_args_t a{};
        a.coll_type              = XCCL_ALLGATHER;
        a.buffer_info.src_buffer = in.data_ptr();
        a.buffer_info.dst_buffer = out.data_ptr();
        a.buffer_info.len        = out.nbytes();
        return run(a, c10d::OpType::_ALLGATHER_BASE, {out}, {in, out});
    }

    c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>> &outs, std::vector<at::Tensor> &ins,
                                             const c10d::AllgatherOptions &opts) override
    {
        TORCH_CHECK(ins.size() == 1 && outs.size() == 1 && static_cast<int>(outs[0].size()) == getSize(), "xccl: bad allgather lists");
        at::Tensor in   = ins[0].contiguous();
        at::Tensor flat = at::empty({static_cast<int64_t>(getSize()) * in.numel()}, in.options());
        auto       w    = _allgather_base(flat, in, opts);
        w->wait();
        for (int r = 0; r < getSize(); r++) {
            outs[0][static_cast<size_t>(r)].copy_(flat.narrow(0, r * in.numel(), in.numel()).view_as(outs[0][static_cast<size_t>(r)]));
        }
        return w;
    }

    c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor &out, at::Tensor &in, const c10d::ReduceScatterOptions &opts) override
    {
        TORCH_CHECK(out.is_contiguous() && in.is_contiguous() && in.numel() == out.numel() * getSize(), "xccl: bad reduce_scatter tensors");
        xccl_coll_op_args_t a{};
        a.coll_type              = XCCL_REDUCE_SCATTER;
        a.buffer_info.src_buffer = in.data_ptr();
        a.buffer_info.dst_buffer = out.data_ptr();
        a.buffer_info.len        = in.nbytes();
        a.reduce_info.dt         = to_dt(in.scalar_type());
        a.reduce_info.op         = to_op(opts.reduceOp);
        a.reduce_info.count      = static_cast<size_t>(out.numel());
        if (opts.reduceOp.op_ == c10d::ReduceOp::AVG) {
            a.field_mask |= XCCL_COLL_OP_ARGS_FIELD_EPILOGUE;
            a.epilogue.scale  = 1.0f / static_cast<float>(getSize());
            a.epilogue.out_dt = XCCL_DT_UNSUPPORTED;
        }
        return run(a, c10d::OpType::_REDUCE_SCATTER_BASE, {out}, {in, out});
    }

    c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor &out, at::Tensor &in, std::vector<int64_t> &out_splits,
                                                 std::vector<int64_t> &in_splits, const c10d::AllToAllOptions &) override
    {
        TORCH_CHECK(out.is_contiguous() && in.is_contiguous(), "xccl: alltoall tensors must be contiguous");
        xccl_coll_op_args_t a{};
        a.buffer_info.src_buffer = in.data_ptr();
        a.buffer_info.dst_buffer = out.data_ptr();
        std::vector<uint32_t> sc, sd, dc, dd;
        if (in_splits.empty() && out_splits.empty()) {
            a.coll_type       = XCCL_ALLTOALL;
            a.buffer_info.len = in.nbytes() / static_cast<size_t>(getSize());
        } else {
            const int64_t row = in.dim() > 0 && in.size(0) > 0 ? in.numel() / in.size(0) : 1;
            uint32_t      so = 0, dof = 0;
            for (int r = 0; r < getSize(); r++) {
                sc.push_back(static_cast<uint32_t>(in_splits[static_cast<size_t>(r)] * row));
                sd.push_back(so);
                so += sc.back();
                dc.push_back(static_cast<uint32_t>(out_splits[static_cast<size_t>(r)] * row));
                dd.push_back(dof);
                dof += dc.back();
            }
            a.coll_type                     = XCCL_ALLTOALLV;
            a.buffer_info.src_counts        = sc.data();
            a.buffer_info.src_displacements = sd.data();
            a.buffer_info.dst_counts        = dc.data();
            a.buffer_info.dst_displacements = dd.data();
            a.buffer_info.src_datatype      = to_dt(in.scalar_type());
            a.buffer_info.dst_datatype      = to_dt(out.scalar_type());
        }
        return run(a, c10d::OpType::ALLTOALL_BASE, {out}, {in, out});
    }

    // ---- list and coalesced forms, built on the flat ones above. Packing and unpacking copies run on the
    // caller's current stream; Work::wait orders that stream after the collective.
    c10::intrusive_ptr<c10d::Work> allreduce_coalesced(std::vector<at::Tensor> &tensors,
                                                       const c10d::AllreduceCoalescedOptions &opts) override
    {
        TORCH_CHECK(!tensors.empty(), "xccl: empty tensor list");
        c10::intrusive_ptr<c10d::Work> w;
        for (auto &t : tensors) {
            std::vector<at::Tensor> one{t};
            w = allreduce(one, opts);
        }
        return w;  // one communication stream: the last one finishing means all have
    }

    c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(std::vector<at::Tensor> &outs, std::vector<at::Tensor> &ins,
                                                                   const c10d::AllgatherOptions &opts) override
    {
        TORCH_CHECK(!ins.empty() && outs.size() == ins.size(), "xccl: bad coalesced allgather lists");
        c10::intrusive_ptr<c10d::Work> w;
        for (size_t i = 0; i < ins.size(); i++) w = _allgather_base(outs[i], ins[i], opts);
        return w;
    }

    c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor> &outs, std::vector<at::Tensor> &ins,
                                                                   const c10d::ReduceScatterOptions &opts) override
    {
        TORCH_CHECK(!ins.empty() && outs.size() == ins.size(), "xccl: bad coalesced reduce_scatter lists");
        c10::intrusive_ptr<c10d::Work> w;
        for (size_t i = 0; i < ins.size(); i++) w = _reduce_scatter_base(outs[i], ins[i], opts);
        return w;
    }

    c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor> &outs, std::vector<std::vector<at::Tensor>> &ins,
                                                  const c10d::ReduceScatterOptions &opts) override
    {
        TORCH_CHECK(outs.size() == 1 && ins.size() == 1 && static_cast<int>(ins[0].size()) == getSize(),
                    "xccl: bad reduce_scatter lists");
        std::vector<at::Tensor> flat_parts;
        for (auto &t : ins[0]) flat_parts.push_back(t.reshape({-1}));
        at::Tensor flat = at::cat(flat_parts);
        at::Tensor out  = outs[0].is_contiguous() ? outs[0] : at::empty_like(outs[0], at::MemoryFormat::Contiguous);
        auto       w    = _reduce_scatter_base(out, flat, opts);
        if (!out.is_same(outs[0])) {
            w->wait();
            outs[0].copy_(out);
        }
        return w;
    }

    // gather / scatter as an alltoallv in which only the root receives / sends
    c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>> &outs, std::vector<at::Tensor> &ins,
                                          const c10d::GatherOptions &opts) override
    {
        TORCH_CHECK(ins.size() == 1, "xccl: one input tensor per gather");
        const int  n = getSize(), root = static_cast<int>(opts.rootRank);
        const bool is_root = getRank() == root;
        TORCH_CHECK(is_root ? (outs.size() == 1 && static_cast<int>(outs[0].size()) == n) : outs.empty(),
                    "xccl: gather output list must have one tensor per rank on the root and be empty elsewhere");
        at::Tensor in   = ins[0].contiguous();
        at::Tensor flat = at::empty({is_root ? static_cast<int64_t>(n) * in.numel() : 1}, in.options());
        std::vector<int64_t> in_splits(static_cast<size_t>(n), 0), out_splits(static_cast<size_t>(n), 0);
        in_splits[static_cast<size_t>(root)] = in.numel();
        if (is_root) std::fill(out_splits.begin(), out_splits.end(), in.numel());
        at::Tensor src = in.reshape({-1});
        auto       w   = alltoallv_flat(flat, src, out_splits, in_splits);
        if (is_root) {
            w->wait();
            for (int r = 0; r < n; r++) {
                at::Tensor &o = outs[0][static_cast<size_t>(r)];
                o.copy_(flat.narrow(0, r * in.numel(), in.numel()).view_as(o));
            }
        }
        return w;
    }

    c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor> &outs, std::vector<std::vector<at::Tensor>> &ins,
                                           const c10d::ScatterOptions &opts) override
    {
        TORCH_CHECK(outs.size() == 1, "xccl: one output tensor per scatter");
        const int  n = getSize(), root = static_cast<int>(opts.rootRank);
        const bool is_root = getRank() == root;
        TORCH_CHECK(is_root ? (ins.size() == 1 && static_cast<int>(ins[0].size()) == n) : ins.empty(),
                    "xccl: scatter input list must have one tensor per rank on the root and be empty elsewhere");
        at::Tensor out = outs[0].is_contiguous() ? outs[0] : at::empty_like(outs[0], at::MemoryFormat::Contiguous);
        at::Tensor flat;
        if (is_root) {
            std::vector<at::Tensor> parts;
            for (auto &t : ins[0]) {
                TORCH_CHECK(t.numel() == out.numel(), "xccl: scatter tensors must have the output's size");
                parts.push_back(t.reshape({-1}));
            }
            flat = at::cat(parts);
        } else {
            flat = at::empty({1}, out.options());
        }
        std::vector<int64_t> in_splits(static_cast<size_t>(n), 0), out_splits(static_cast<size_t>(n), 0);
        out_splits[static_cast<size_t>(root)] = out.numel();
        if (is_root) std::fill(in_splits.begin(), in_splits.end(), out.numel());
        at::Tensor dst = out.view({-1});
        auto       w   = alltoallv_flat(dst, flat, out_splits, in_splits);
        if (!out.is_same(outs[0])) {
            w->wait();
            outs[0].copy_(out);
        }
        return w;
    }

    c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor> &outs, std::vector<at::Tensor> &ins,
                                            const c10d::AllToAllOptions &) override
    {
        const int n = getSize();
        TORCH_CHECK(static_cast<int>(outs.size()) == n && static_cast<int>(ins.size()) == n, "xccl: alltoall lists need one tensor per rank");
        std::vector<int64_t>    in_splits, out_splits;
        std::vector<at::Tensor> parts;
        int64_t                 out_total = 0;
        for (int r = 0; r < n; r++) {
            TORCH_CHECK(ins[static_cast<size_t>(r)].scalar_type() == ins[0].scalar_type() &&
                        outs[static_cast<size_t>(r)].scalar_type() == ins[0].scalar_type(), "xccl: alltoall tensors must share a dtype");
            in_splits.push_back(ins[static_cast<size_t>(r)].numel());
            out_splits.push_back(outs[static_cast<size_t>(r)].numel());
            parts.push_back(ins[static_cast<size_t>(r)].reshape({-1}));
            out_total += out_splits.back();
        }
        at::Tensor src = at::cat(parts);
        if (src.numel() == 0) src = at::empty({1}, ins[0].options());
        at::Tensor dst = at::empty({std::max<int64_t>(out_total, 1)}, outs[0].options());
        auto       w   = alltoallv_flat(dst, src, out_splits, in_splits);
        w->wait();
        int64_t off = 0;
        for (int r = 0; r < n; r++) {
            at::Tensor &o = outs[static_cast<size_t>(r)];
            if (o.numel() > 0) o.copy_(dst.narrow(0, off, o.numel()).view_as(o));
            off += o.numel();
        }
        return w;
    }

    c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions &) override
    {
        xccl_coll_op_args_t a{};
        a.coll_type         = XCCL_BARRIER;
        xccl_coll_req_h req = nullptr;
        check(xccl_collective_init(&a, &req, team_), "xccl_collective_init");
        check(xccl_collective_post(req), "xccl_collective_post");
        check(xccl_collective_wait(req), "xccl_collective_wait");
        check(xccl_collective_finalize(req), "xccl_collective_finalize");
        auto work = c10::make_intrusive<WorkXccl>(c10d::OpType::BARRIER, std::vector<at::Tensor>{}, false);
        work->complete();
        return work;
    }

    void shutdown() override { reap(true); }

    // Point-to-point on NCCL p2p (pipeline stages). A two-rank communicator per peer is created by both sides at
    // their first send/recv with each other, bootstrapped through the store under a pair-specific key prefix.
    c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor> &tensors, int dstRank, int /*tag*/) override
    {
        return p2p(tensors, dstRank, true);
    }
    c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor> &tensors, int srcRank, int /*tag*/) override
    {
        return p2p(tensors, srcRank, false);
    }

private:
    // element-count splits over flat 1-D tensors
    c10::intrusive_ptr<c10d::Work> alltoallv_flat(at::Tensor &out, at::Tensor &in, std::vector<int64_t> &out_splits,
                                                  std::vector<int64_t> &in_splits)
    {
        xccl_coll_op_args_t a{};
        a.buffer_info.src_buffer = in.data_ptr();
        a.buffer_info.dst_buffer = out.data_ptr();
        std::vector<uint32_t> sc, sd, dc, dd;
        uint32_t              so = 0, dof = 0;
        for (int r = 0; r < getSize(); r++) {
            sc.push_back(static_cast<uint32_t>(in_splits[static_cast<size_t>(r)]));
            sd.push_back(so);
            so += sc.back();
            dc.push_back(static_cast<uint32_t>(out_splits[static_cast<size_t>(r)]));
            dd.push_back(dof);
            dof += dc.back();
        }
        a.coll_type                     = XCCL_ALLTOALLV;
        a.buffer_info.src_counts        = sc.data();
        a.buffer_info.src_displacements = sd.data();
        a.buffer_info.dst_counts        = dc.data();
        a.buffer_info.dst_displacements = dd.data();
        a.buffer_info.src_datatype      = to_dt(in.scalar_type());
        a.buffer_info.dst_datatype      = to_dt(out.scalar_type());
        return run(a, c10d::OpType::ALLTOALL, {out}, {in, out});
    }

    struct PairComm {
        StoreOob               state;
        xccl_oob_collectives_t oob{};
        void                  *comm = nullptr;
    };

    PairComm &pair_comm(int peer)
    {
        auto it = pairs_.find(peer);
        if (it != pairs_.end()) return *it->second;
        const int me = getRank(), lo = std::min(me, peer), hi = std::max(me, peer);
        auto      pc = std::make_unique<PairComm>();
        pc->state    = StoreOob{oob_state_.store, me == lo ? 0 : 1, 2, {}, "p2p/" + std::to_string(lo) + "-" + std::to_string(hi) + "/"};
        pc->oob.allgather    = store_allgather;
        pc->oob.req_test     = store_test;
        pc->oob.req_free     = store_free;
        pc->oob.coll_context = &pc->state;
        pc->oob.rank         = pc->state.rank;
        pc->oob.size         = 2;
        check(xccl_p2p_comm_create(&pc->oob, &pc->comm), "xccl_p2p_comm_create");
        return *pairs_.emplace(peer, std::move(pc)).first->second;
    }

    c10::intrusive_ptr<c10d::Work> p2p(std::vector<at::Tensor> &tensors, int peer, bool is_send)
    {
        TORCH_CHECK(tensors.size() == 1, "xccl: send/recv take one tensor");
        at::Tensor &t = tensors[0];
        TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "xccl: send/recv need a contiguous CUDA tensor");
        TORCH_CHECK(peer != getRank() && peer >= 0 && peer < getSize(), "xccl: bad peer rank");
        c10::cuda::CUDAGuard dev_guard(t.device());
        PairComm            &pc   = pair_comm(peer);
        auto                 work = c10::make_intrusive<WorkXccl>(is_send ? c10d::OpType::SEND : c10d::OpType::RECV,
                                                  std::vector<at::Tensor>{t}, true);
        auto                 cur  = c10::cuda::getCurrentCUDAStream();
        auto                 comm = comm_stream(t.device().index());
        at::cuda::CUDAEvent  ready;
        ready.record(cur);
        ready.block(comm);
        c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), comm);
        const int    peer_in_pair = pc.state.rank == 0 ? 1 : 0;
        const size_t bytes        = static_cast<size_t>(t.numel()) * t.element_size();
        check(is_send ? xccl_p2p_send(pc.comm, t.data_ptr(), bytes, peer_in_pair, comm.stream())
                      : xccl_p2p_recv(pc.comm, t.data_ptr(), bytes, peer_in_pair, comm.stream()),
              is_send ? "xccl_p2p_send" : "xccl_p2p_recv");
        c10::cuda::CUDAStreamGuard guard(comm);
        work->complete();
        return work;
    }

    c10::cuda::CUDAStream comm_stream(c10::DeviceIndex dev)
    {
        auto it = streams_.find(dev);
        if (it == streams_.end()) it = streams_.emplace(dev, c10::cuda::getStreamFromPool(true, dev)).first;
        return it->second;
    }
    // finished requests are finalized lazily; `all` waits for everything (shutdown)
    void reap(bool all)
    {
        for (size_t i = 0; i < pending_.size();) {
            xccl_status_t st = all ? xccl_collective_wait(pending_[i]) : xccl_collective_test(pending_[i]);
            if (st != XCCL_INPROGRESS) {
                TORCH_CHECK(st == XCCL_OK, "xccl: a collective failed: ", xccl_status_str(st));
                xccl_collective_finalize(pending_[i]);
                pending_.erase(pending_.begin() + static_cast<long>(i));
            } else {
                i++;
            }
        }
    }

    StoreOob                                       oob_state_;
    xccl_oob_collectives_t                         oob_{};
    xccl_lib_h                                     lib_  = nullptr;
    xccl_context_h                                 ctx_  = nullptr;
    xccl_team_h                                    team_ = nullptr;
    std::map<c10::DeviceIndex, c10::cuda::CUDAStream> streams_;
    std::vector<xccl_coll_req_h>                   pending_;
    std::map<int, std::unique_ptr<PairComm>>       pairs_;
};

c10::intrusive_ptr<c10d::Backend> create_backend(const c10::intrusive_ptr<c10d::Store> &store, int rank, int size,
                                                 const std::chrono::duration<float> &)
{
    return c10::make_intrusive<ProcessGroupXccl>(store, rank, size);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
    m.doc() = "c10d backend over the xccl C API";
    m.def("create_backend", &create_backend);
    m.def("allreduce_fused",
          [](const c10::intrusive_ptr<c10d::Backend> &b, at::Tensor in, at::Tensor out, double scale) {
              auto *pg = dynamic_cast<ProcessGroupXccl *>(b.get());
              TORCH_CHECK(pg != nullptr, "not a b200xccl backend");
              return pg->allreduce_fused(std::move(in), std::move(out), scale);
          });
    m.def("empty_symmetric", [](const c10::intrusive_ptr<c10d::Backend> &b, int64_t nbytes, int dev) {
        auto *pg = dynamic_cast<ProcessGroupXccl *>(b.get());
        TORCH_CHECK(pg != nullptr, "not a b200xccl backend");
        return pg->empty_symmetric(nbytes, static_cast<c10::DeviceIndex>(dev));
    });
    m.def("free_symmetric", [](const c10::intrusive_ptr<c10d::Backend> &b, const at::Tensor &t) {
        auto *pg = dynamic_cast<ProcessGroupXccl *>(b.get());
        TORCH_CHECK(pg != nullptr, "not a b200xccl backend");
        pg->free_symmetric(t);
    });
    m.def("coll_tl", [](const c10::intrusive_ptr<c10d::Backend> &b, int coll, bool cuda) {
        auto *pg = dynamic_cast<ProcessGroupXccl *>(b.get());
        TORCH_CHECK(pg != nullptr, "not a b200xccl backend");
        return pg->coll_tl(coll, cuda);
    });
}
