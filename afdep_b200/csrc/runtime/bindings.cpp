// Host runtime of one rank's Buffer and its Python bindings.
//
// NativeBuffer owns the symmetric heap, the device-local scratch of the rank's role, the
// mapped-host status block, and launches the exchange kernels on the caller's current
// CUDA stream.  Nothing here synchronises with the device except construction, destroy()
// and the optional exact-count path of worker_receive; epochs live in device memory, so a
// captured CUDA graph replays an exchange without host involvement.
//
// Counterpart of the reference's ElasticBuffer host class (csrc/elastic/buffer.hpp:19-1347)
// and pybind module (csrc/python_api.cpp), without NCCL, JIT or a comm-stream detour.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <chrono>
#include <cstdlib>
#include <memory>
#include <mutex>
#include <thread>

#include "afdep/aux_api.h"
#include "afdep/expert_gemm_api.h"
#include "afdep/gemm_api.h"
#include "afdep/kernels.h"
#include "afdep/quant_api.h"
#include "afdep/route_layout_api.h"
#include "driver.hpp"
#include "heap.hpp"
#include "stream_memops.hpp"

namespace py = pybind11;

namespace afdep {

namespace {

const char* code_name(int code) {
    switch (code) {
        case kOk: return "ok";
        case kTimeoutCounts: return "timeout waiting for a source's counts";
        case kTimeoutRecord: return "timeout waiting for a record";
        case kTimeoutReply: return "timeout waiting for a reply row";
        case kTimeoutLookback: return "timeout in the dispatch look-back";
        case kTimeoutBarrier: return "timeout in barrier";
        case kTimeoutAux: return "timeout in an auxiliary primitive";
        case kBadRoute: return "illegal route";
        case kBadIndex: return "computed index out of bounds";
        default: return "unknown";
    }
}

SymmetricHeap::Mode parse_mode(const std::string& m) {
    if (m == "vmm") return SymmetricHeap::Mode::kVmmFd;
    if (m == "ipc") return SymmetricHeap::Mode::kCudaIpc;
    if (m == "plain") return SymmetricHeap::Mode::kPlain;
    throw std::invalid_argument("heap mode must be 'vmm', 'ipc' or 'plain'");
}

}  // namespace

namespace {

// Tensor map of a row-major [rows, cols] matrix with 128-byte-swizzled boxes of `box_rows`
// rows by 128 bytes, the tile shape the grouped GEMM's shared-memory descriptors expect.
CUtensorMap make_tile_map(const void* base, int64_t rows, int64_t cols, int elem_bytes, int box_rows) {
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * (cuuint64_t)elem_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    drv_check(AFDEP_DRV(cuTensorMapEncodeTiled)(&map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
              "cuTensorMapEncodeTiled");
    return map;
}

}  // namespace

// SM clock in kHz, asked once per device: this attribute is a live driver query (milliseconds),
// not a cached property, so it must stay off the launch path.
int device_khz(int device) {
    static std::mutex mu;
    static int cache[64] = {};
    std::lock_guard<std::mutex> lock(mu);
    if (device < 0 || device >= 64) device = 0;
    if (cache[device] == 0) {
        int khz = 0;
        rt_check(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device), "device attribute");
        cache[device] = khz > 0 ? khz : 1000000;
    }
    return cache[device];
}

// The device's GEMM error word, after raising for any failure an earlier launch left in it.  A
// kernel whose bounded wait ran out sets the word and returns with its output incomplete; the
// next GEMM call on that device (or gemm_check) reports it.
int* checked_gemm_error_word(int device) {
    const GemmErrorWord w = gemm_error_word(device);
    TORCH_CHECK(w.host != nullptr, "could not allocate the GEMM error word");
    if (*w.host != 0) {
        *w.host = 0;
        throw std::runtime_error("an earlier expert GEMM on this device gave up on a bounded wait; its output is incomplete");
    }
    return w.device;
}

class NativeBuffer {
public:
    NativeBuffer(int rank, int ffn, int attn, int hidden, int top_k, int num_experts, int capacity, bool fp8,
                 int alignment, int num_sms, int collect_sms, int ffn_sms, double gpu_timeout_s,
                 int64_t aux_bytes, const std::string& heap_mode, bool bounds_check, int p2p_inflight, int scale_packs)
        : rank_(rank), num_sms_(num_sms), collect_sms_(collect_sms), ffn_sms_(ffn_sms), p2p_inflight_(p2p_inflight) {
        TORCH_CHECK(p2p_inflight >= 1 && p2p_inflight <= 64, "p2p_inflight must be between 1 and 64");
        TORCH_CHECK(ffn + attn <= kMaxRanks, "the native transport supports at most ", kMaxRanks, " ranks");
        TORCH_CHECK(num_experts <= kMaxExperts && num_experts / ffn <= kMaxExpertsLocal, "too many experts");
        TORCH_CHECK(top_k <= kMaxTopK, "top_k too large");
        rt_check(cudaGetDevice(&device_), "cudaGetDevice");
        TORCH_CHECK(scale_packs >= 0 && scale_packs <= hidden / 128, "scale_packs must be between 0 and hidden / 128");
        geo_ = make_geometry(ffn, attn, hidden, top_k, num_experts, capacity, fp8 ? 1 : 0, alignment, (size_t)aux_bytes, scale_packs);
        is_ffn_ = rank < ffn;
        role_rank_ = is_ffn_ ? rank : rank - ffn;
        const size_t bytes = is_ffn_ ? geo_.f_bytes : geo_.a_bytes;
        heap_ = std::make_unique<SymmetricHeap>(device_, bytes, parse_mode(heap_mode));
        rt_check(cudaMemset(heap_->local(), 0, bytes), "cudaMemset(heap)");

        int sms = 0, smem = 0, khz = 0;
        rt_check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device_), "device attribute");
        rt_check(cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device_), "device attribute");
        rt_check(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device_), "device attribute");
        device_sms_ = sms;
        max_smem_ = smem;
        if (num_sms_ <= 0 || num_sms_ > sms) num_sms_ = sms;
        if (collect_sms_ <= 0 || collect_sms_ > sms) collect_sms_ = sms;
        if (ffn_sms_ <= 0 || ffn_sms_ > sms) ffn_sms_ = sms;
        rt_check(configure_kernels(max_smem_), "cudaFuncSetAttribute");
        rt_check(configure_aux(), "cudaFuncSetAttribute");

        // status block and host-count mailbox in mapped pinned memory
        rt_check(cudaHostAlloc(&host_block_, kHostBlockBytes, cudaHostAllocMapped), "cudaHostAlloc");
        std::memset(host_block_, 0, kHostBlockBytes);
        void* dev_view = nullptr;
        rt_check(cudaHostGetDevicePointer(&dev_view, host_block_, 0), "cudaHostGetDevicePointer");

        auto i32 = torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, device_);
        flags_ = torch::zeros({64}, i32);   // poison words, epochs, tickets
        int* fl = flags_.data_ptr<int>();
        ctx_.g = geo_;
        ctx_.rank = rank;
        ctx_.role_rank = role_rank_;
        for (int i = 0; i < kMaxRanks; ++i) ctx_.peer[i] = nullptr;
        ctx_.peer[rank] = static_cast<char*>(heap_->local());
        ctx_.status = static_cast<Status*>(dev_view);
        ctx_.poison = fl;                       // words 0..3
        ctx_.budget = (long long)(gpu_timeout_s * 1000.0 * (double)khz);
        ctx_.bounds_check = bounds_check ? 1 : 0;
        ctx_.trace = nullptr;
        barrier_epoch_ = reinterpret_cast<unsigned*>(fl + 8);
        if (is_ffn_) {
            fws_.epoch = reinterpret_cast<unsigned*>(fl + 16);    // 3 words
            fws_.ticket = reinterpret_cast<unsigned*>(fl + 24);   // 2 words
            scratch_ = torch::zeros({(int64_t)attn * geo_.experts_local + attn + 1 + geo_.experts_local + 8}, i32);
            int* s = scratch_.data_ptr<int>();
            fws_.row_base = s;
            fws_.rec_prefix = s + (size_t)attn * geo_.experts_local;
            fws_.ends = fws_.rec_prefix + attn + 1;
            fws_.host_counts = reinterpret_cast<int*>(static_cast<char*>(dev_view) + kHostCountsOff);
        } else {
            aws_.epoch = reinterpret_cast<unsigned*>(fl + 16);    // 2 words
            aws_.ticket = reinterpret_cast<unsigned*>(fl + 24);
            const int64_t ncols = ffn + num_experts;
            agg_ = torch::zeros({(int64_t)max_dispatch_ctas() * ncols}, torch::TensorOptions().dtype(torch::kInt64).device(torch::kCUDA, device_));
            scratch_ = torch::zeros({(int64_t)capacity * (2 * top_k + ffn) + max_dispatch_ctas()}, i32);
            int* s = scratch_.data_ptr<int>();
            aws_.chunk_done = reinterpret_cast<unsigned*>(s + (size_t)capacity * (2 * top_k + ffn));
            aws_.agg = reinterpret_cast<unsigned long long*>(agg_.data_ptr<int64_t>());
            aws_.route_e = s;
            aws_.route_pos = s + (size_t)capacity * top_k;
            aws_.tok_slot = s + (size_t)capacity * top_k * 2;
        }
        rt_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    }

    ~NativeBuffer() {
        try {
            destroy();
        } catch (...) {
        }
    }

    // ---- heap exchange --------------------------------------------------------------
    int64_t heap_bytes() const { return (int64_t)heap_->bytes(); }
    int64_t mapped_bytes() const { return (int64_t)heap_->mapped_bytes(); }
    int64_t local_ptr() const { return reinterpret_cast<int64_t>(heap_->local()); }
    int export_fd() { return heap_->export_fd(); }
    py::bytes export_ipc() { return py::bytes(heap_->export_ipc()); }
    void import_peer_fd(int peer, int fd, int64_t mapped) {
        check_peer(peer);
        ctx_.peer[peer] = static_cast<char*>(heap_->import_fd(fd, (size_t)mapped));
    }
    void import_peer_ipc(int peer, const std::string& handle) {
        check_peer(peer);
        ctx_.peer[peer] = static_cast<char*>(heap_->import_ipc(handle));
    }
    void set_peer_ptr(int peer, int64_t ptr) {   // loopback world: all heaps live in this process
        check_peer(peer);
        ctx_.peer[peer] = reinterpret_cast<char*>(ptr);
    }
    bool peers_complete() const {
        for (int i = 0; i < geo_.world; ++i)
            if (!ctx_.peer[i]) return false;
        return true;
    }

    // ---- collective-ish operations ---------------------------------------------------
    void barrier() {
        live();
        rt_check(launch_barrier(ctx_, barrier_epoch_, stream()), "barrier launch");
    }

    void source_dispatch(const torch::Tensor& x, const c10::optional<torch::Tensor>& x_scale,
                         const torch::Tensor& ids, const torch::Tensor& weights) {
        live();
        TORCH_CHECK(!is_ffn_, "source_dispatch runs on attention ranks");
        const int T = (int)x.size(0);
        TORCH_CHECK(T <= geo_.capacity, "more tokens than the registered capacity");
        TORCH_CHECK(reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0, "x must be 16-byte aligned");
        DispatchArgs a{};
        a.x = x.data_ptr();
        if (ids.scalar_type() == torch::kInt32)
            a.ids32 = ids.data_ptr<int>();
        else
            a.ids = reinterpret_cast<const long long*>(ids.data_ptr<int64_t>());
        a.weights = weights.data_ptr<float>();
        a.T = T;
        static const int flag_mode = std::getenv("AFDEP_FLAG_MODE") ? std::atoi(std::getenv("AFDEP_FLAG_MODE")) : 0;
        a.flag_mode = flag_mode;
        if (geo_.fp8) {
            TORCH_CHECK(x_scale.has_value(), "FP8 dispatch needs scales");
            a.x_scale = x_scale->data_ptr<float>();
            a.ss0 = x_scale->stride(0);
            a.ss1 = x_scale->stride(1);
        }
        const LaunchShape s = dispatch_shape(geo_, T, num_sms_, max_smem_);
        rt_check(launch_dispatch(ctx_, aws_, a, s, stream()), "dispatch launch");
        ++launches_;
    }

    torch::Tensor source_collect(int64_t T) {
        live();
        TORCH_CHECK(!is_ffn_, "source_collect runs on attention ranks");
        auto out = torch::empty({T, geo_.hidden}, torch::TensorOptions().dtype(torch::kBFloat16).device(torch::kCUDA, device_));
        const LaunchShape s = collect_shape(geo_, (int)T, collect_sms_, max_smem_);
        rt_check(launch_collect(ctx_, aws_, out.data_ptr(), (int)T, s, stream()), "collect launch");
        ++launches_;
        return out;
    }

    // Returns (recv_x, recv_scale or None, recv_weights, psum, host_counts, recv_src).
    py::tuple worker_receive(int64_t rows_bound, bool read_host_counts, double cpu_timeout_s, bool col_major_scale) {
        live();
        TORCH_CHECK(is_ffn_, "worker_receive runs on FFN ranks");
        auto dev = torch::TensorOptions().device(torch::kCUDA, device_);
        const int EL = geo_.experts_local;
        auto psum = torch::empty({EL}, dev.dtype(torch::kInt32));
        ReceiveArgs r{};
        r.psum = psum.data_ptr<int>();
        r.expert_stats = expert_stats_.defined() ? reinterpret_cast<long long*>(expert_stats_.data_ptr<int64_t>()) : nullptr;
        std::vector<int64_t> host_counts;
        int64_t rows = rows_bound;
        if (read_host_counts) {
            r.write_host_counts = 1;
            r.rows_cap = (int)rows_bound;
            volatile int* hc = reinterpret_cast<volatile int*>(static_cast<char*>(host_block_) + kHostCountsOff);
            const int want = (int)(++host_seq_);
            rt_check(launch_ffn_layout(ctx_, fws_, r, stream()), "layout launch");
            ++launches_;
            int seen = 0;
            {
                py::gil_scoped_release nogil;
                const auto t0 = std::chrono::steady_clock::now();
                while (true) {
                    seen = hc[EL];
                    if (seen == want || seen == -want) break;
                    const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
                    if (dt > cpu_timeout_s) break;
                    std::this_thread::yield();
                }
            }
            if (seen != want) {
                failed_ = true;
                throw std::runtime_error(seen == -want ? "worker_receive: the device gave up waiting for source counts: " + status_text()
                                                       : "worker_receive: timed out on the host waiting for receive counts");
            }
            rows = 0;
            for (int e = 0; e < EL; ++e) {
                host_counts.push_back(hc[e]);
                rows += hc[e];
            }
            r.layout_ready = 1;
            r.write_host_counts = 0;
        }
        auto recv_x = torch::empty({rows, geo_.hidden}, dev.dtype(geo_.fp8 ? torch::kFloat8_e4m3fn : torch::kBFloat16));
        auto recv_w = torch::empty({rows}, dev.dtype(torch::kFloat32));
        auto recv_src = torch::empty({rows, 2}, dev.dtype(torch::kInt32));
        c10::optional<torch::Tensor> recv_scale;
        if (geo_.fp8) {
            const int64_t sg = geo_.scale_groups;
            if (col_major_scale) {
                const int64_t ld = (rows + 3) / 4 * 4;
                recv_scale = torch::empty_strided({rows, sg}, {1, ld > 0 ? ld : 4}, dev.dtype(torch::kFloat32));
            } else {
                recv_scale = torch::empty({rows, sg}, dev.dtype(torch::kFloat32));
            }
            r.recv_scale = recv_scale->data_ptr<float>();
            r.rs0 = recv_scale->stride(0);
            r.rs1 = recv_scale->stride(1);
        }
        r.recv_x = recv_x.data_ptr();
        r.recv_w = recv_w.data_ptr<float>();
        r.recv_src = recv_src.data_ptr<int>();
        r.rows_cap = (int)rows;
        const LaunchShape s = receive_shape(geo_, ffn_sms_, max_smem_);
        rt_check(launch_receive(ctx_, fws_, r, s, stream()), "receive launch");
        ++launches_;
        py::object scale_obj = recv_scale.has_value() ? py::cast(*recv_scale) : py::none();
        return py::make_tuple(recv_x, scale_obj, recv_w, psum, host_counts, recv_src);
    }

    // Running total of rows received per local expert, summed on the device by the receive
    // path from now on (int64 [experts_local]); the tensor stays valid until destroy().  The
    // reference offers the same counter as an optional dispatch argument
    // (csrc/elastic/buffer.hpp:740-748).
    torch::Tensor enable_expert_stats() {
        TORCH_CHECK(!destroyed_, "buffer is closed");
        TORCH_CHECK(is_ffn_, "expert statistics are kept on FFN ranks");
        if (!expert_stats_.defined())
            expert_stats_ = torch::zeros({geo_.experts_local}, torch::TensorOptions().dtype(torch::kInt64).device(torch::kCUDA, device_));
        return expert_stats_;
    }

    void worker_reply(const torch::Tensor& rows) {
        live();
        TORCH_CHECK(is_ffn_, "worker_reply runs on FFN ranks");
        TORCH_CHECK(reinterpret_cast<uintptr_t>(rows.data_ptr()) % 16 == 0, "rows must be 16-byte aligned");
        const LaunchShape s = reply_shape(geo_, ffn_sms_, max_smem_);
        rt_check(launch_reply(ctx_, fws_, rows.data_ptr(), (int)rows.size(0), s, stream()), "reply launch");
        ++launches_;
    }


    // Receive, experts and reply of one exchange without the expert-major copy of the received
    // rows: a one-CTA layout pass, then the gate|up GEMM that indexes the wire records as they land
    // and gathers its A rows straight from the staging region (SwiGLU in the epilogue), the down
    // projection times the routing weight, and the reply kernel.  FP8 payloads need FP8 weights
    // with power-of-two block scales; BF16 payloads need BF16 weights.
    // Returns (psum, recv_weights, recv_src, rows sent back).
    py::tuple worker_mlp_fused(const torch::Tensor& w_gate_up, const c10::optional<torch::Tensor>& w_gate_up_scale,
                               const torch::Tensor& w_down, const c10::optional<torch::Tensor>& w_down_scale, int64_t rows_bound) {
        live();
        TORCH_CHECK(is_ffn_, "worker_mlp_fused runs on FFN ranks");
        const int EL = geo_.experts_local, H = geo_.hidden;
        const bool fp8 = geo_.fp8 != 0;
        const auto wdt = fp8 ? torch::kFloat8_e4m3fn : torch::kBFloat16;
        TORCH_CHECK(w_gate_up.is_cuda() && w_gate_up.dim() == 3 && w_gate_up.is_contiguous() && w_gate_up.scalar_type() == wdt &&
                        w_gate_up.size(0) == EL && w_gate_up.size(2) == H && w_gate_up.size(1) % 256 == 0,
                    "w_gate_up: [experts_local, 2*intermediate, hidden] in the payload's dtype");
        const int64_t I = w_gate_up.size(1) / 2;
        TORCH_CHECK(w_down.is_cuda() && w_down.dim() == 3 && w_down.is_contiguous() && w_down.scalar_type() == wdt && w_down.size(0) == EL &&
                        w_down.size(1) == H && w_down.size(2) == I && I % 128 == 0,
                    "w_down: [experts_local, hidden, intermediate] in the payload's dtype");
        TORCH_CHECK(geo_.alignment % 128 == 0, "the fused expert path needs expert_alignment to be a multiple of 128");
        if (fp8) {
            TORCH_CHECK(w_gate_up_scale.has_value() && w_down_scale.has_value(), "FP8 experts need their block scales");
            TORCH_CHECK(w_gate_up_scale->scalar_type() == torch::kFloat32 && w_gate_up_scale->is_contiguous() &&
                            w_gate_up_scale->numel() == (int64_t)EL * (2 * I / 128) * (H / 128),
                        "w_gate_up_scale: fp32 [experts_local, 2I/128, H/128]");
            TORCH_CHECK(w_down_scale->scalar_type() == torch::kFloat32 && w_down_scale->is_contiguous() &&
                            w_down_scale->numel() == (int64_t)EL * (H / 128) * (I / 128),
                        "w_down_scale: fp32 [experts_local, H/128, I/128]");
        }
        const int64_t rows = rows_bound;
        auto dev = torch::TensorOptions().device(torch::kCUDA, device_);
        auto psum = torch::empty({EL}, dev.dtype(torch::kInt32));
        auto recv_w = torch::empty({rows}, dev.dtype(torch::kFloat32));
        auto recv_src = torch::empty({rows, 2}, dev.dtype(torch::kInt32));
        auto row_rec = torch::empty({rows}, dev.dtype(torch::kInt32));
        const int64_t n_tiles = rows / 128 + 1;
        if (!tile_cnt_.defined() || tile_cnt_.numel() < n_tiles) tile_cnt_ = torch::zeros({n_tiles}, dev.dtype(torch::kInt32));
        auto out = torch::empty({rows, H}, dev.dtype(torch::kBFloat16));
        cudaStream_t st = stream();

        ReceiveArgs r{};
        r.psum = psum.data_ptr<int>();
        r.expert_stats = expert_stats_.defined() ? reinterpret_cast<long long*>(expert_stats_.data_ptr<int64_t>()) : nullptr;
        r.rows_cap = (int)rows;
        r.tile_cnt = reinterpret_cast<unsigned*>(tile_cnt_.data_ptr<int>());
        r.tile_cnt_n = (int)n_tiles;
        rt_check(launch_ffn_layout(ctx_, fws_, r, st), "layout launch");
        ++launches_;

        int* err = checked_gemm_error_word(device_);
        ExpertGemmArgs g{};
        g.rows = (int)rows;
        g.N = (int)(2 * I);
        g.K = H;
        g.experts = EL;
        g.alignment = geo_.alignment;
        g.ends = psum.data_ptr<int>();
        g.mx = fp8 ? 1 : 0;
        g.budget = ctx_.budget;
        g.a_rows = reinterpret_cast<const unsigned char*>(heap_->local()) + geo_.f_stage;
        g.a_pitch = geo_.rec_bytes;
        g.row_rec = row_rec.data_ptr<int>();
        g.a_scale_off = fp8 ? geo_.payload_bytes : -1;
        g.a_scale_packed = (fp8 && geo_.scale_groups != geo_.hidden / 128) ? 1 : 0;      // the Buffer carries packed exponent words
        g.w_scale = fp8 ? w_gate_up_scale->data_ptr<float>() : nullptr;
        g.swiglu = 1;
        g.ldc = (int)I;
        g.error = err;
        torch::Tensor h, h_scale;
        if (fp8) {
            h = torch::empty({rows, I}, dev.dtype(torch::kFloat8_e4m3fn));
            h_scale = torch::empty({rows, I / 128}, dev.dtype(torch::kFloat32));
            g.out_q = static_cast<unsigned char*>(h.data_ptr());
            g.out_q_scale = h_scale.data_ptr<float>();
            g.oqs0 = h_scale.stride(0);
            g.oqs1 = h_scale.stride(1);
        } else {
            h = torch::empty({rows, I}, dev.dtype(torch::kBFloat16));
            g.out = reinterpret_cast<__nv_bfloat16*>(h.data_ptr());
        }
        FusedReceive fr{};
        fr.enabled = 1;
        fr.c = ctx_;
        fr.ws = fws_;
        fr.row_rec = row_rec.data_ptr<int>();
        fr.recv_w = recv_w.data_ptr<float>();
        fr.recv_src = recv_src.data_ptr<int>();
        fr.tile_cnt = reinterpret_cast<unsigned*>(tile_cnt_.data_ptr<int>());
        fr.rows_cap = (int)rows;
        const int elem = fp8 ? 1 : 2;
        const int grid = ffn_sms_ < device_sms_ ? ffn_sms_ : device_sms_;
        const CUtensorMap map_gu = make_tile_map(w_gate_up.data_ptr(), (int64_t)EL * 2 * I, H, elem, 256);
        rt_check(launch_expert_gemm(map_gu, map_gu, g, /*gather=*/true, fr, grid, st), "fused gate/up GEMM launch");
        ++launches_;

        ExpertGemmArgs d{};
        d.rows = (int)rows;
        d.N = H;
        d.K = (int)I;
        d.experts = EL;
        d.alignment = geo_.alignment;
        d.ends = psum.data_ptr<int>();
        d.mx = fp8 ? 1 : 0;
        d.budget = ctx_.budget;
        d.a_scale_off = -1;
        if (fp8) {
            d.a_scale = h_scale.data_ptr<float>();
            d.a_scale_s0 = h_scale.stride(0);
            d.a_scale_s1 = h_scale.stride(1);
            d.w_scale = w_down_scale->data_ptr<float>();
        }
        d.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
        d.ldc = H;
        d.row_scale = recv_w.data_ptr<float>();
        d.error = err;
        const CUtensorMap map_h = make_tile_map(h.data_ptr(), rows, I, elem, 128);
        const CUtensorMap map_dn = make_tile_map(w_down.data_ptr(), (int64_t)EL * H, I, elem, 256);
        FusedReceive none{};
        rt_check(launch_expert_gemm(map_h, map_dn, d, /*gather=*/false, none, device_sms_, st), "down GEMM launch");
        ++launches_;

        const LaunchShape s = reply_shape(geo_, ffn_sms_, max_smem_);
        rt_check(launch_reply(ctx_, fws_, out.data_ptr(), (int)rows, s, st), "reply launch");
        ++launches_;
        return py::make_tuple(psum, recv_w, recv_src, out);
    }

    // ---- status -----------------------------------------------------------------------
    py::dict status() {
        const volatile Status* s = static_cast<const volatile Status*>(host_block_);
        py::dict d;
        const int code = s->code;
        d["code"] = code;
        d["text"] = std::string(code_name(code));
        d["kernel"] = s->kernel;
        d["rank"] = s->rank;
        d["peer"] = s->peer;
        d["epoch"] = s->epoch;
        d["expected"] = s->expected;
        d["observed"] = s->observed;
        d["detail0"] = s->detail0;
        d["detail1"] = s->detail1;
        d["fatal"] = code != kOk && code != kBadRoute;
        return d;
    }
    int status_code() const { return static_cast<const volatile Status*>(host_block_)->code; }

    // After a non-fatal report (an illegal route): forget it so the next one is recorded.
    void clear_status() {
        rt_check(cudaStreamSynchronize(stream()), "cudaStreamSynchronize");
        std::memset(host_block_, 0, sizeof(Status));
        rt_check(cudaMemsetAsync(ctx_.poison, 0, 4 * sizeof(int), stream()), "cudaMemsetAsync");
        rt_check(cudaStreamSynchronize(stream()), "cudaStreamSynchronize");
    }
    int bad_routes() {
        int v = 0;
        rt_check(cudaMemcpy(&v, ctx_.poison + 2, sizeof(int), cudaMemcpyDeviceToHost), "cudaMemcpy");
        return v;
    }

    // ---- secondary primitives on the auxiliary region ----------------------------------------
    int64_t aux_data_bytes() const { return geo_.aux_bytes > (size_t)kAuxSignalBytes ? (int64_t)(geo_.aux_bytes - kAuxSignalBytes) : 0; }
    // Largest all-gather contribution (two slot sets, by gather parity) and largest message
    // (a ring of p2p_inflight slots per source rank).
    int64_t aux_slot_bytes() const { return aux_data_bytes() / (2 * geo_.world) / 16 * 16; }
    int64_t p2p_slot_bytes() const { return aux_data_bytes() / ((int64_t)geo_.world * p2p_inflight_) / 16 * 16; }
    int p2p_inflight() const { return p2p_inflight_; }

    // View of this rank's auxiliary data area as bytes (peers write into it).
    torch::Tensor aux_view() {
        live();
        auto* base = static_cast<unsigned char*>(heap_->local()) + geo_.aux_off + kAuxSignalBytes;
        return torch::from_blob(base, {aux_data_bytes()}, torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, device_));
    }
    // Snapshot of this rank's 24 signal words (gather flags, send flags, credits), for diagnostics.
    torch::Tensor aux_signals() {
        live();
        auto* base = static_cast<unsigned char*>(heap_->local()) + geo_.aux_off;
        auto view = torch::from_blob(base, {24}, torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, device_));
        return view.clone();
    }
    void allgather_push(const torch::Tensor& t) {
        live();
        const size_t bytes = check_aux_tensor(t, aux_slot_bytes());
        rt_check(launch_allgather_push(ctx_, aux_seq(), t.data_ptr(), bytes, (size_t)aux_slot_bytes(), aux_ctas(bytes), stream()), "all-gather launch");
        ++launches_;
    }
    // The same all-gather without an SM: one copy-engine transfer per peer, then one batched
    // stream memory operation that writes this gather's number into every peer's flag word.
    // The number comes from a host-side count of completed gathers, so this form cannot be
    // captured into a CUDA graph; once a capture has contained the kernel form, the count is
    // re-read from the device (one stream synchronisation) before every use.
    void allgather_push_copy(const torch::Tensor& t) {
        live();
        const size_t bytes = check_aux_tensor(t, aux_slot_bytes());
        cudaStream_t s = stream();
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        rt_check(cudaStreamIsCapturing(s, &cap), "cudaStreamIsCapturing");
        TORCH_CHECK(cap == cudaStreamCaptureStatusNone, "the copy-engine all-gather cannot be captured into a CUDA graph");
        if (gather_in_graph_) {     // replays advance the device count behind the host's back
            rt_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
            rt_check(cudaMemcpy(&gathers_done_, aux_seq().gather, sizeof(unsigned), cudaMemcpyDeviceToHost), "cudaMemcpy");
        }
        const size_t slot = (size_t)aux_slot_bytes();
        const size_t set = (size_t)((gathers_done_ + 1u) & 1u) * geo_.world;       // slot set of this gather's parity
        std::vector<StreamWrite32> flags;
        for (int p = 0; p < geo_.world; ++p) {
            char* aux = ctx_.peer[p] + geo_.aux_off;
            rt_check(cudaMemcpyAsync(aux + kAuxSignalBytes + (set + (size_t)rank_) * slot, t.data_ptr(), bytes, cudaMemcpyDeviceToDevice, s),
                     "all-gather peer copy");
            flags.push_back({aux + sizeof(uint32_t) * (size_t)rank_, gathers_done_ + 1u});
        }
        stream_write32_batch(s, flags);
    }
    // Waits for every rank's contribution and returns a copy of the gathered bytes
    // [world, nbytes]: the heap slots are free for the gather after next as soon as this returns.
    torch::Tensor allgather_wait(int64_t nbytes) {
        live();
        TORCH_CHECK(nbytes >= 0 && nbytes <= aux_slot_bytes(), "gathered size exceeds the slot");
        cudaStream_t s = stream();
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        rt_check(cudaStreamIsCapturing(s, &cap), "cudaStreamIsCapturing");
        auto out = torch::empty({geo_.world, nbytes}, torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, device_));
        if (cap != cudaStreamCaptureStatusNone)
            gather_in_graph_ = true;       // replays advance the device count behind the host's back
        else
            ++gathers_done_;
        // The copy-out reads the gather's parity from the device count, so it is right in graph replays too.
        rt_check(launch_allgather_wait(ctx_, aux_seq(), s), "all-gather wait launch");
        rt_check(launch_allgather_copy_out(ctx_, aux_seq(), out.data_ptr(), (size_t)nbytes, (size_t)aux_slot_bytes(), s), "all-gather copy launch");
        launches_ += 2;
        return out;
    }
    void p2p_send(const torch::Tensor& t, int dst) {
        live();
        check_peer(dst);
        const size_t bytes = check_aux_tensor(t, p2p_slot_bytes());
        rt_check(launch_p2p_send(ctx_, aux_seq(), dst, t.data_ptr(), bytes, (size_t)p2p_slot_bytes(), p2p_inflight_, aux_ctas(bytes), stream()),
                 "send launch");
        ++launches_;
    }
    void p2p_recv(torch::Tensor& t, int src) {
        live();
        check_peer(src);
        const size_t bytes = check_aux_tensor(t, p2p_slot_bytes());
        rt_check(launch_p2p_recv(ctx_, aux_seq(), src, t.data_ptr(), bytes, (size_t)p2p_slot_bytes(), p2p_inflight_, aux_ctas(bytes), stream()),
                 "recv launch");
        ++launches_;
    }
    torch::Tensor fetch_rows(const torch::Tensor& idx, int64_t rows_per_rank, int64_t row_bytes) {
        live();
        TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == torch::kInt64 && idx.is_contiguous(), "idx: contiguous CUDA int64");
        TORCH_CHECK(row_bytes % 16 == 0 && rows_per_rank > 0 && rows_per_rank * row_bytes <= aux_data_bytes(), "table shard does not fit the auxiliary region");
        const int64_t n = idx.numel();
        auto out = torch::empty({n, row_bytes}, torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, device_));
        if (n == 0) return out;
        const int ctas = (int)std::min<int64_t>(num_sms_, (n + 7) / 8);
        rt_check(launch_fetch_rows(ctx_, reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()), (int)n, (int)rows_per_rank,
                                   (int)row_bytes, out.data_ptr(), ctas, stream()), "fetch launch");
        ++launches_;
        return out;
    }

    // Per-CTA time stamps of the exchange kernels: int64 [kTraceRows][kTraceCtas][4] in
    // nanoseconds of the GPU's global timer; pass enable=false to switch tracing off again.
    torch::Tensor trace(bool enable) {
        if (!enable) {
            ctx_.trace = nullptr;
            return trace_;
        }
        if (!trace_.defined())
            trace_ = torch::zeros({kTraceRows, kTraceCtas, 4}, torch::TensorOptions().dtype(torch::kInt64).device(torch::kCUDA, device_));
        ctx_.trace = reinterpret_cast<unsigned long long*>(trace_.data_ptr<int64_t>());
        return trace_;
    }

    // Test hook: overwrite the payload regions of this rank's heap (wire records and reply rows on
    // an FFN rank) with 0xFF bytes -- NaN in BF16, e4m3 and fp32 -- on the current stream.  Flags,
    // counts and barrier words are left alone.  Only meaningful while no exchange is in flight on
    // any rank; a stale read in a later exchange then shows up as NaN instead of plausible data.
    void poison_payload() {
        live();
        if (!is_ffn_) return;
        auto* base = static_cast<unsigned char*>(heap_->local());
        rt_check(cudaMemsetAsync(base + geo_.f_stage, 0xFF, geo_.f_bytes - geo_.f_stage, stream()), "cudaMemsetAsync");
    }

    // Debugging knob: CTA budget of the next dispatches, not clamped to the device (up to the
    // size of the look-back scratch).  A budget the GPU cannot hold at once makes the cooperative
    // dispatch launch fail on the host instead of timing out on the device.
    void set_dispatch_ctas(int n) {
        TORCH_CHECK(n >= 1 && n <= max_dispatch_ctas(), "dispatch CTA budget out of range");
        num_sms_ = n;
    }

    int64_t launches() const { return launches_; }
    int resolved_num_sms() const { return num_sms_; }
    int device_sms() const { return device_sms_; }
    int64_t record_bytes() const { return geo_.rec_bytes; }

    void destroy() {
        if (destroyed_) return;
        destroyed_ = true;
        cudaSetDevice(device_);
        cudaDeviceSynchronize();
        flags_ = torch::Tensor();
        scratch_ = torch::Tensor();
        agg_ = torch::Tensor();
        trace_ = torch::Tensor();
        expert_stats_ = torch::Tensor();
        tile_cnt_ = torch::Tensor();
        heap_->release();
        if (host_block_) cudaFreeHost(host_block_);
        host_block_ = nullptr;
    }

private:
    AuxSeq aux_seq() {
        int* fl = flags_.data_ptr<int>();
        AuxSeq q{};
        q.gather = reinterpret_cast<unsigned*>(fl + 32);
        q.sent = reinterpret_cast<unsigned*>(fl + 40);
        q.received = reinterpret_cast<unsigned*>(fl + 48);
        q.ticket = reinterpret_cast<unsigned*>(fl + 56);
        return q;
    }
    size_t check_aux_tensor(const torch::Tensor& t, int64_t slot) const {
        TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "tensor must be a contiguous CUDA tensor");
        const size_t bytes = (size_t)t.numel() * t.element_size();
        TORCH_CHECK(bytes % 16 == 0 && reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, "tensor must be 16-byte aligned and sized");
        TORCH_CHECK((int64_t)bytes <= slot, "tensor larger than its slot of the auxiliary region (raise aux_bytes)");
        return bytes;
    }
    // One CTA (one SM's copy engine) per 64 KB, up to the whole device: these primitives run on their
    // own, not beside a compute kernel, and a remote store takes microseconds to drain, so the link is
    // only filled when many SMs have stores in flight.
    int aux_ctas(size_t bytes) const {
        const int want = (int)((bytes + 65535) / 65536);
        return want < 1 ? 1 : (want > device_sms_ ? device_sms_ : want);
    }

    static constexpr size_t kHostBlockBytes = 8192;
    static constexpr size_t kHostCountsOff = 1024;

    cudaStream_t stream() const { return at::cuda::getCurrentCUDAStream(device_).stream(); }
    void live() const {
        TORCH_CHECK(!destroyed_, "buffer is closed");
        TORCH_CHECK(peers_complete(), "peer heaps have not been connected");
    }
    void check_peer(int peer) const { TORCH_CHECK(peer >= 0 && peer < geo_.world, "peer out of range"); }
    std::string status_text() {
        const volatile Status* s = static_cast<const volatile Status*>(host_block_);
        return std::string(code_name(s->code)) + " (rank " + std::to_string(s->rank) + ", peer " + std::to_string(s->peer) + ")";
    }

    int rank_, role_rank_ = 0, device_ = 0, device_sms_ = 0, max_smem_ = 0;
    int num_sms_, collect_sms_, ffn_sms_, p2p_inflight_;
    bool is_ffn_ = false, destroyed_ = false, failed_ = false;
    Geometry geo_{};
    RankCtx ctx_{};
    AttnWs aws_{};
    FfnWs fws_{};
    unsigned* barrier_epoch_ = nullptr;
    std::unique_ptr<SymmetricHeap> heap_;
    void* host_block_ = nullptr;
    torch::Tensor flags_, scratch_, agg_, trace_;
    int64_t host_seq_ = 0, launches_ = 0;
    torch::Tensor expert_stats_;      // optional running per-expert row totals
    torch::Tensor tile_cnt_;          // fused expert path: rows indexed per 128-row tile
    unsigned gathers_done_ = 0;       // all-gathers waited for outside graph capture
    bool gather_in_graph_ = false;    // an all-gather wait has been captured into a graph
};

// Deterministic routing layout of one source (see kernels/layout.cu).  Returns
// (route_e [T,K], route_pos [T,K], tok_slot [T,F], counts [F+E]) as int32 tensors.
py::tuple route_layout(const torch::Tensor& ids, int64_t num_experts, int64_t ffn_ranks) {
    TORCH_CHECK(ids.is_cuda() && ids.dim() == 2 && ids.scalar_type() == torch::kInt64 && ids.is_contiguous(),
                "ids must be a contiguous CUDA int64 [tokens, top_k] tensor");
    TORCH_CHECK(ffn_ranks >= 1 && ffn_ranks <= kMaxRanks && num_experts % ffn_ranks == 0 && num_experts <= kMaxExperts,
                "unsupported expert geometry");
    const int64_t T = ids.size(0), K = ids.size(1);
    TORCH_CHECK(K >= 1 && K <= kMaxTopK, "top_k out of range");
    c10::cuda::CUDAGuard guard(ids.device());
    auto i32 = torch::TensorOptions().dtype(torch::kInt32).device(ids.device());
    auto scratch = torch::zeros({(int64_t)route_layout_scratch_bytes((int)num_experts, (int)ffn_ranks)},
                                torch::TensorOptions().dtype(torch::kUInt8).device(ids.device()));
    auto route_e = torch::empty({T, K}, i32);
    auto route_pos = torch::empty({T, K}, i32);
    auto tok_slot = torch::empty({T, ffn_ranks}, i32);
    auto counts = torch::empty({ffn_ranks + num_experts}, i32);
    const int khz = device_khz(ids.get_device());
    rt_check(launch_route_layout(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), (int)T, (int)K,
                                 (int)num_experts, (int)ffn_ranks, scratch.data_ptr(), route_e.data_ptr<int>(),
                                 route_pos.data_ptr<int>(), tok_slot.data_ptr<int>(), counts.data_ptr<int>(),
                                 (long long)khz * 1000ll * 5ll, at::cuda::getCurrentCUDAStream().stream()),
             "route_layout launch");
    return py::make_tuple(route_e, route_pos, tok_slot, counts);
}



// out[rows, N or N/2] = A[rows, K] x W[e][N, K]^T per expert segment, on tcgen05.
// a: bf16 or e4m3 [rows, K]; w: same dtype [experts, N, K]; ends: int32 [experts].
// Returns the BF16 output, or with quantize_out (FP8 operands + swiglu) the pair
// (e4m3 output [rows, N/2], fp32 scales [rows, N/256]).
py::object grouped_gemm(const torch::Tensor& a, const torch::Tensor& w, const torch::Tensor& ends, int64_t alignment,
                        bool swiglu, const c10::optional<torch::Tensor>& row_scale,
                        const c10::optional<torch::Tensor>& a_scale, const c10::optional<torch::Tensor>& w_scale,
                        const c10::optional<torch::Tensor>& out_opt, int64_t ctas, bool quantize_out) {
    TORCH_CHECK(a.is_cuda() && w.is_cuda() && ends.is_cuda(), "grouped_gemm needs CUDA tensors");
    TORCH_CHECK(a.dim() == 2 && w.dim() == 3 && a.is_contiguous() && w.is_contiguous(), "a [rows,K], w [experts,N,K], contiguous");
    TORCH_CHECK(a.scalar_type() == w.scalar_type(), "a and w must have the same dtype");
    const bool fp8 = a.scalar_type() == torch::kFloat8_e4m3fn;
    TORCH_CHECK(fp8 || a.scalar_type() == torch::kBFloat16, "bf16 or float8_e4m3fn operands");
    const int64_t rows = a.size(0), K = a.size(1), E = w.size(0), N = w.size(1);
    TORCH_CHECK(w.size(2) == K && K % 128 == 0 && N % 128 == 0, "K and N must be multiples of 128");
    TORCH_CHECK(alignment % 128 == 0, "expert_alignment must be a multiple of 128 for the grouped GEMM");
    TORCH_CHECK(ends.scalar_type() == torch::kInt32 && ends.numel() == E && E <= kMaxExpertsLocal, "ends: int32 [experts]");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(a.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(w.data_ptr()) % 16 == 0,
                "operands must be 16-byte aligned");
    c10::cuda::CUDAGuard guard(a.device());
    const int64_t ldc = swiglu ? N / 2 : N;
    torch::Tensor out, out_q, out_q_scale;
    if (quantize_out) {
        TORCH_CHECK(fp8 && swiglu && N % 256 == 0 && !out_opt.has_value(),
                    "quantize_out needs FP8 operands, swiglu, N a multiple of 256 and no preallocated out");
        out_q = torch::empty({rows, ldc}, torch::TensorOptions().dtype(torch::kFloat8_e4m3fn).device(a.device()));
        out_q_scale = torch::empty({rows, ldc / 128}, torch::TensorOptions().dtype(torch::kFloat32).device(a.device()));
    } else {
        out = out_opt.has_value() ? *out_opt
                                  : torch::empty({rows, ldc}, torch::TensorOptions().dtype(torch::kBFloat16).device(a.device()));
        TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.is_contiguous() && out.size(0) == rows && out.size(1) == ldc,
                    "out must be contiguous bf16 [rows, N or N/2]");
    }
    const py::object result = quantize_out ? py::object(py::make_tuple(out_q, out_q_scale)) : py::cast(out);
    GroupedGemmArgs g{};
    g.rows = (int)rows;
    g.N = (int)N;
    g.K = (int)K;
    g.experts = (int)E;
    g.alignment = (int)alignment;
    g.ends = ends.data_ptr<int>();
    g.out = quantize_out ? nullptr : reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
    if (quantize_out) {
        g.out_q = static_cast<unsigned char*>(out_q.data_ptr());
        g.out_q_scale = out_q_scale.data_ptr<float>();
        g.oqs0 = out_q_scale.stride(0);
        g.oqs1 = out_q_scale.stride(1);
    }
    g.ldc = (int)ldc;
    g.swiglu = swiglu ? 1 : 0;
    g.row_scale = row_scale.has_value() ? row_scale->data_ptr<float>() : nullptr;
    g.fp8 = fp8 ? 1 : 0;
    if (fp8) {
        TORCH_CHECK(a_scale.has_value() && w_scale.has_value(), "FP8 operands need a_scale [rows, K/128] and w_scale [experts, N/128, K/128]");
        TORCH_CHECK(a_scale->scalar_type() == torch::kFloat32 && a_scale->size(0) == rows && a_scale->size(1) == K / 128, "a_scale shape");
        TORCH_CHECK(w_scale->scalar_type() == torch::kFloat32 && w_scale->is_contiguous() && w_scale->numel() == E * (N / 128) * (K / 128),
                    "w_scale shape");
        g.a_scale = a_scale->data_ptr<float>();
        g.a_scale_s0 = a_scale->stride(0);
        g.a_scale_s1 = a_scale->stride(1);
        g.w_scale = w_scale->data_ptr<float>();
    }
    if (rows == 0) return result;
    const int elem = fp8 ? 1 : 2;
    int sms = 0;
    rt_check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, a.get_device()), "device attribute");
    const int grid = ctas > 0 ? (int)ctas : sms;
    g.error = checked_gemm_error_word(a.get_device());
    const CUtensorMap map_a = make_tile_map(a.data_ptr(), rows, K, elem, 128);
    const CUtensorMap map_w = make_tile_map(w.data_ptr(), E * N, K, elem, 256);
    rt_check(launch_grouped_gemm(map_a, map_w, g, grid, at::cuda::getCurrentCUDAStream().stream()), "grouped_gemm launch");
    return result;
}


// The self-feeding expert GEMM (kernels/expert_gemm.cu) as a stand-alone operation.
//   a          dense form: [rows, K] bf16 / e4m3.  Gathered form (row_index given): any contiguous
//              2-D tensor whose row i starts with the K operand elements of "record" i; uint8 rows
//              may carry the row's K/128 fp32 scales at byte offset a_scale_offset.
//   row_index  optional int32 [rows]: record of every row of the row space (< 0: a row of zeros)
//   FP8 operands need power-of-two scales (a_scale [rows, K/128] or in-record; w_scale).
// Returns BF16 [rows, N or N/2], or with quantize_out (e4m3 [rows, N/2], fp32 power-of-two scales [rows, N/256]).
py::object expert_gemm(const torch::Tensor& a, const torch::Tensor& w, const torch::Tensor& ends, int64_t alignment, bool swiglu,
                       const c10::optional<torch::Tensor>& row_scale, const c10::optional<torch::Tensor>& a_scale,
                       const c10::optional<torch::Tensor>& w_scale, const c10::optional<torch::Tensor>& out_opt, int64_t ctas,
                       bool quantize_out, const c10::optional<torch::Tensor>& row_index, int64_t a_scale_offset, bool a_scale_packed) {
    TORCH_CHECK(a.is_cuda() && w.is_cuda() && ends.is_cuda(), "expert_gemm needs CUDA tensors");
    TORCH_CHECK(a.dim() == 2 && w.dim() == 3 && a.is_contiguous() && w.is_contiguous(), "a 2-D, w [experts,N,K], contiguous");
    const bool fp8 = w.scalar_type() == torch::kFloat8_e4m3fn;
    TORCH_CHECK(fp8 || w.scalar_type() == torch::kBFloat16, "bf16 or float8_e4m3fn weights");
    const bool gather = row_index.has_value();
    const int64_t E = w.size(0), N = w.size(1), K = w.size(2);
    const int elem = fp8 ? 1 : 2;
    int64_t rows;
    if (gather) {
        TORCH_CHECK(row_index->is_cuda() && row_index->scalar_type() == torch::kInt32 && row_index->is_contiguous() && row_index->dim() == 1,
                    "row_index: contiguous int32 [rows] on the GPU");
        rows = row_index->numel();
        TORCH_CHECK(a.scalar_type() == w.scalar_type() || a.scalar_type() == torch::kUInt8, "gathered rows: the weights' dtype, or raw uint8 records");
        TORCH_CHECK(a.size(1) * a.element_size() >= K * elem && (a.size(1) * a.element_size()) % 16 == 0, "records shorter than K, or pitch not a multiple of 16 bytes");
    } else {
        TORCH_CHECK(a.scalar_type() == w.scalar_type() && a.size(1) == K, "a must be [rows, K] of the weights' dtype");
        rows = a.size(0);
    }
    TORCH_CHECK(K % 128 == 0 && N % 128 == 0, "K and N must be multiples of 128");
    TORCH_CHECK(alignment % 128 == 0, "expert_alignment must be a multiple of 128 for the expert GEMM");
    TORCH_CHECK(ends.scalar_type() == torch::kInt32 && ends.numel() == E && E <= kMaxExpertsLocal, "ends: int32 [experts]");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(a.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(w.data_ptr()) % 16 == 0, "operands must be 16-byte aligned");
    c10::cuda::CUDAGuard guard(w.device());
    const int64_t ldc = swiglu ? N / 2 : N;
    torch::Tensor out, out_q, out_q_scale;
    if (quantize_out) {
        TORCH_CHECK(fp8 && swiglu && N % 256 == 0 && !out_opt.has_value(), "quantize_out needs FP8 operands, swiglu, N a multiple of 256 and no preallocated out");
        out_q = torch::empty({rows, ldc}, torch::TensorOptions().dtype(torch::kFloat8_e4m3fn).device(w.device()));
        out_q_scale = torch::empty({rows, ldc / 128}, torch::TensorOptions().dtype(torch::kFloat32).device(w.device()));
    } else {
        out = out_opt.has_value() ? *out_opt : torch::empty({rows, ldc}, torch::TensorOptions().dtype(torch::kBFloat16).device(w.device()));
        TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.is_contiguous() && out.size(0) == rows && out.size(1) == ldc, "out must be contiguous bf16 [rows, N or N/2]");
    }
    const py::object result = quantize_out ? py::object(py::make_tuple(out_q, out_q_scale)) : py::cast(out);
    ExpertGemmArgs g{};
    g.rows = (int)rows;
    g.N = (int)N;
    g.K = (int)K;
    g.experts = (int)E;
    g.alignment = (int)alignment;
    g.ends = ends.data_ptr<int>();
    g.mx = fp8 ? 1 : 0;
    g.budget = (long long)device_khz(w.get_device()) * 1000ll * 10ll;
    g.a_scale_off = -1;
    if (gather) {
        g.a_rows = static_cast<const unsigned char*>(a.data_ptr());
        g.a_pitch = a.size(1) * a.element_size();
        g.row_rec = row_index->data_ptr<int>();
    }
    if (fp8) {
        TORCH_CHECK(w_scale.has_value() && w_scale->scalar_type() == torch::kFloat32 && w_scale->is_contiguous() &&
                        w_scale->numel() == E * (N / 128) * (K / 128), "w_scale: fp32 [experts, N/128, K/128]");
        g.w_scale = w_scale->data_ptr<float>();
        const int64_t words = (K / 128 + 3) / 4;        // packed form: four exponent bytes to a word
        if (a_scale.has_value() && a_scale->scalar_type() == torch::kInt32) {
            TORCH_CHECK(a_scale->is_cuda() && a_scale->dim() == 2 && a_scale->size(0) == rows && a_scale->size(1) == words,
                        "packed a_scale: int32 [rows, ceil(K/512)]");
            g.a_scale = reinterpret_cast<const float*>(a_scale->data_ptr<int>());
            g.a_scale_s0 = a_scale->stride(0);
            g.a_scale_s1 = a_scale->stride(1);
            g.a_scale_packed = 1;
        } else if (a_scale.has_value()) {
            TORCH_CHECK(a_scale->scalar_type() == torch::kFloat32 && a_scale->size(0) == rows && a_scale->size(1) == K / 128, "a_scale: fp32 [rows, K/128]");
            g.a_scale = a_scale->data_ptr<float>();
            g.a_scale_s0 = a_scale->stride(0);
            g.a_scale_s1 = a_scale->stride(1);
        } else {
            TORCH_CHECK(gather && a_scale_offset >= K && a_scale_offset % 16 == 0 &&
                            a_scale_offset + (a_scale_packed ? words * 4 : words * 16) <= g.a_pitch,
                        "FP8 operands need a_scale, or gathered records with the scales (fp32 padded to whole 16-byte groups, or packed words) "
                        "at a 16-byte aligned a_scale_offset");
            g.a_scale_off = (int)a_scale_offset;
            g.a_scale_packed = a_scale_packed ? 1 : 0;
        }
    }
    g.out = quantize_out ? nullptr : reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
    if (quantize_out) {
        g.out_q = static_cast<unsigned char*>(out_q.data_ptr());
        g.out_q_scale = out_q_scale.data_ptr<float>();
        g.oqs0 = out_q_scale.stride(0);
        g.oqs1 = out_q_scale.stride(1);
    }
    g.ldc = (int)ldc;
    g.swiglu = swiglu ? 1 : 0;
    g.row_scale = row_scale.has_value() ? row_scale->data_ptr<float>() : nullptr;
    if (rows == 0) return result;
    g.error = checked_gemm_error_word(w.get_device());
    int sms = 0;
    rt_check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, w.get_device()), "device attribute");
    const int grid = ctas > 0 ? (int)ctas : sms;
    const CUtensorMap map_w = make_tile_map(w.data_ptr(), E * N, K, elem, 256);
    const CUtensorMap map_a = gather ? map_w : make_tile_map(a.data_ptr(), rows, K, elem, 128);
    FusedReceive fr{};
    rt_check(launch_expert_gemm(map_a, map_w, g, gather, fr, grid, at::cuda::getCurrentCUDAStream().stream()), "expert_gemm launch");
    return result;
}

// (e4m3 [rows, K], fp32 scales [rows, K/128]) from bf16 rows; `limit` (optional int32 device
// tensor, e.g. recv_count_psum[-1:]) marks the first row that need not be quantised.
py::tuple quantize_rows_fp8(const torch::Tensor& x, const c10::optional<torch::Tensor>& limit, bool pow2) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == torch::kBFloat16 && x.is_contiguous(), "x: contiguous CUDA bf16 [rows, K]");
    const int64_t rows = x.size(0), K = x.size(1);
    TORCH_CHECK(K % 128 == 0, "K must be a multiple of 128");
    c10::cuda::CUDAGuard guard(x.device());
    auto q = torch::empty({rows, K}, torch::TensorOptions().dtype(torch::kFloat8_e4m3fn).device(x.device()));
    auto scale = torch::empty({rows, K / 128}, torch::TensorOptions().dtype(torch::kFloat32).device(x.device()));
    const int* lim = nullptr;
    if (limit.has_value()) {
        TORCH_CHECK(limit->is_cuda() && limit->scalar_type() == torch::kInt32 && limit->numel() >= 1, "limit: int32 CUDA tensor");
        lim = limit->data_ptr<int>();
    }
    int sms = 0;
    rt_check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, x.get_device()), "device attribute");
    rt_check(launch_quantize_rows(x.data_ptr(), q.data_ptr(), scale.data_ptr<float>(), (int)rows, (int)K, scale.stride(0), scale.stride(1), lim, pow2,
                                  sms * 8, at::cuda::getCurrentCUDAStream().stream()),
             "quantize launch");
    return py::make_tuple(q, scale);
}

}  // namespace afdep

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    using afdep::NativeBuffer;
    m.doc() = "afdep_b200 native runtime (sm_100a)";
    m.attr("max_ranks") = afdep::kMaxRanks;
    m.def("vmm_supported", [](int device) { return afdep::SymmetricHeap::vmm_supported(device); });
    // What this library was compiled as and against; the doctor prints it.  Counterpart of the
    // reference module's version and architecture queries (csrc/python_api.cpp:26-56).
    m.def("build_info", [] {
        py::dict d;
        int runtime = 0, driver = 0;
        cudaRuntimeGetVersion(&runtime);
        if (cudaDriverGetVersion(&driver) != cudaSuccess) cudaGetLastError();
        d["arch"] = "sm_100a";
        d["cuda_compiled"] = CUDART_VERSION;
        d["cuda_runtime"] = runtime;
        d["cuda_driver"] = driver;
        d["topk_index_dtype"] = "int64 or int32 (Buffer option topk_idx_bits)";
        d["max_ranks"] = afdep::kMaxRanks;
        d["trace_ctas"] = afdep::kTraceCtas;
        d["stream_memops"] = true;
        return d;
    });
    // Heap layout and launch shapes as plain numbers, for checks that need no GPU: offsets,
    // alignments and shared-memory budgets are pure functions of the configuration.
    m.def("geometry", [](int ffn, int attn, int hidden, int top_k, int num_experts, int capacity, bool fp8, int alignment, int64_t aux_bytes,
                         int scale_packs) {
        const afdep::Geometry g = afdep::make_geometry(ffn, attn, hidden, top_k, num_experts, capacity, fp8 ? 1 : 0, alignment, (size_t)aux_bytes, scale_packs);
        py::dict d;
        d["payload_bytes"] = g.payload_bytes;
        d["scale_bytes"] = g.scale_bytes;
        d["meta_bytes"] = g.meta_bytes;
        d["meta_off"] = g.meta_off;
        d["rec_bytes"] = g.rec_bytes;
        d["row_bytes"] = g.row_bytes;
        d["experts_local"] = g.experts_local;
        d["cnt_stride"] = afdep::cnt_stride(g);
        d["ctrl_bytes"] = (int64_t)g.ctrl_bytes;
        d["aux_off"] = (int64_t)g.aux_off;
        d["aux_bytes"] = (int64_t)g.aux_bytes;
        d["f_cnt"] = (int64_t)g.f_cnt;
        d["f_slot_flag"] = (int64_t)g.f_slot_flag;
        d["f_stage"] = (int64_t)g.f_stage;
        d["f_reply"] = (int64_t)g.f_reply;
        d["f_bytes"] = (int64_t)g.f_bytes;
        d["a_reply_flag"] = (int64_t)g.a_reply_flag;
        d["a_bytes"] = (int64_t)g.a_bytes;
        return d;
    },
          py::arg("ffn"), py::arg("attn"), py::arg("hidden"), py::arg("top_k"), py::arg("num_experts"), py::arg("capacity"), py::arg("fp8"),
          py::arg("alignment"), py::arg("aux_bytes"), py::arg("scale_packs") = 0);
    m.def("launch_shapes", [](int ffn, int attn, int hidden, int top_k, int num_experts, int capacity, bool fp8, int alignment, int tokens,
                              int num_sms, int collect_sms, int ffn_sms, int max_smem) {
        const afdep::Geometry g = afdep::make_geometry(ffn, attn, hidden, top_k, num_experts, capacity, fp8 ? 1 : 0, alignment, 0);
        auto pack = [](const afdep::LaunchShape& s) { return py::make_tuple(s.ctas, s.warps, s.smem_bytes); };
        py::dict d;
        d["dispatch"] = pack(afdep::dispatch_shape(g, tokens, num_sms, max_smem));
        d["receive"] = pack(afdep::receive_shape(g, ffn_sms, max_smem));
        d["reply"] = pack(afdep::reply_shape(g, ffn_sms, max_smem));
        d["collect"] = pack(afdep::collect_shape(g, tokens, collect_sms, max_smem));
        return d;
    });
    m.def("grouped_gemm", &afdep::grouped_gemm, py::arg("a"), py::arg("w"), py::arg("ends"), py::arg("alignment"),
          py::arg("swiglu") = false, py::arg("row_scale") = py::none(), py::arg("a_scale") = py::none(),
          py::arg("w_scale") = py::none(), py::arg("out") = py::none(), py::arg("ctas") = 0, py::arg("quantize_out") = false);
    m.def("expert_gemm", &afdep::expert_gemm, py::arg("a"), py::arg("w"), py::arg("ends"), py::arg("alignment"), py::arg("swiglu") = false,
          py::arg("row_scale") = py::none(), py::arg("a_scale") = py::none(), py::arg("w_scale") = py::none(), py::arg("out") = py::none(),
          py::arg("ctas") = 0, py::arg("quantize_out") = false, py::arg("row_index") = py::none(), py::arg("a_scale_offset") = -1,
          py::arg("a_scale_packed") = false);
    // True (and cleared) if an expert GEMM on this device gave up on a bounded wait since the last check.
    m.def("gemm_check", [](int device) {
        const afdep::GemmErrorWord w = afdep::gemm_error_word(device);
        if (w.host == nullptr || *w.host == 0) return false;
        *w.host = 0;
        return true;
    });
    m.def("quantize_rows_fp8", &afdep::quantize_rows_fp8, py::arg("x"), py::arg("limit") = py::none(), py::arg("pow2") = false);
    m.def("route_layout", &afdep::route_layout, py::arg("ids"), py::arg("num_experts"), py::arg("ffn_ranks"));
    py::class_<NativeBuffer>(m, "NativeBuffer")
        .def(py::init<int, int, int, int, int, int, int, bool, int, int, int, int, double, int64_t, const std::string&, bool, int, int>(),
             py::arg("rank"), py::arg("ffn"), py::arg("attn"), py::arg("hidden"), py::arg("top_k"), py::arg("num_experts"),
             py::arg("capacity"), py::arg("fp8"), py::arg("alignment"), py::arg("num_sms"), py::arg("collect_sms"),
             py::arg("ffn_sms"), py::arg("gpu_timeout_s"), py::arg("aux_bytes"), py::arg("heap_mode"), py::arg("bounds_check"), py::arg("p2p_inflight") = 4,
             py::arg("scale_packs") = 0)
        .def("heap_bytes", &NativeBuffer::heap_bytes)
        .def("mapped_bytes", &NativeBuffer::mapped_bytes)
        .def("local_ptr", &NativeBuffer::local_ptr)
        .def("export_fd", &NativeBuffer::export_fd)
        .def("export_ipc", &NativeBuffer::export_ipc)
        .def("import_peer_fd", &NativeBuffer::import_peer_fd)
        .def("import_peer_ipc", &NativeBuffer::import_peer_ipc)
        .def("set_peer_ptr", &NativeBuffer::set_peer_ptr)
        .def("peers_complete", &NativeBuffer::peers_complete)
        .def("barrier", &NativeBuffer::barrier)
        .def("source_dispatch", &NativeBuffer::source_dispatch)
        .def("source_collect", &NativeBuffer::source_collect)
        .def("worker_receive", &NativeBuffer::worker_receive)
        .def("worker_reply", &NativeBuffer::worker_reply)
        .def("worker_mlp_fused", &NativeBuffer::worker_mlp_fused)
        .def("status", &NativeBuffer::status)
        .def("status_code", &NativeBuffer::status_code)
        .def("clear_status", &NativeBuffer::clear_status)
        .def("bad_routes", &NativeBuffer::bad_routes)
        .def("trace", &NativeBuffer::trace)
        .def("aux_data_bytes", &NativeBuffer::aux_data_bytes)
        .def("aux_slot_bytes", &NativeBuffer::aux_slot_bytes)
        .def("p2p_slot_bytes", &NativeBuffer::p2p_slot_bytes)
        .def("p2p_inflight", &NativeBuffer::p2p_inflight)
        .def("aux_view", &NativeBuffer::aux_view)
        .def("aux_signals", &NativeBuffer::aux_signals)
        .def("allgather_push", &NativeBuffer::allgather_push)
        .def("enable_expert_stats", &NativeBuffer::enable_expert_stats)
        .def("allgather_push_copy", &NativeBuffer::allgather_push_copy)
        .def("allgather_wait", &NativeBuffer::allgather_wait)
        .def("p2p_send", &NativeBuffer::p2p_send)
        .def("p2p_recv", &NativeBuffer::p2p_recv)
        .def("fetch_rows", &NativeBuffer::fetch_rows)
        .def("set_dispatch_ctas", &NativeBuffer::set_dispatch_ctas)
        .def("poison_payload", &NativeBuffer::poison_payload)
        .def("launches", &NativeBuffer::launches)
        .def("resolved_num_sms", &NativeBuffer::resolved_num_sms)
        .def("device_sms", &NativeBuffer::device_sms)
        .def("record_bytes", &NativeBuffer::record_bytes)
        .def("destroy", &NativeBuffer::destroy);
}
