// Source-level stand-in for the subset of the TTNN / tt-metalium C++ API that tt-perf's executors, examples,
// tests and benchmarks call (autograd/{dynamic,static,traced}/*.hpp, autograd/common.hpp, examples/*.cpp,
// verify/*.cpp, bench/**.cpp). Every operation forwards to the C ABI of include/b200_ttperf.h; this header adds no
// arithmetic of its own. The include paths the reference uses (<ttnn/operations/matmul/matmul.hpp>, ...) are thin
// headers next to this one that include it.
//
// Conventions kept from the reference:
//  * `Tensor` is a cheap-to-copy handle to ref-counted device (or host) storage; op results are returned by value;
//  * ops are queued asynchronously, in order, on the device's command queue (here: the context's CUDA stream);
//    `Finish`, `Synchronize`, `Tensor::cpu()` and a blocking `execute_trace` are the only synchronisation points;
//  * failures surface as exceptions derived from std::exception (the C ABI's status codes are converted here).
// Layout tags (TILE / ROW_MAJOR) and memory configs are accepted and carried, but storage is always row-major.
#pragma once

#include <algorithm>
#include <array>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <initializer_list>
#include <iostream>
#include <memory>
#include <numeric>
#include <optional>
#include <ostream>
#include <random>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#include "../b200_ttperf.h"
#include "../fmt/core.h"

// ---------------------------------------------------------------------------------------------------------------------
// bfloat16 (tt-metalium/bfloat16.hpp): global class, constructible from float, convertible back
// ---------------------------------------------------------------------------------------------------------------------
class bfloat16 {
    uint16_t bits_ = 0;

public:
    bfloat16() = default;
    bfloat16(float f) {
        uint32_t u;
        std::memcpy(&u, &f, 4);
        if ((u & 0x7fffffffu) > 0x7f800000u) {
            bits_ = static_cast<uint16_t>((u >> 16) | 0x40);  // quiet NaN
        } else {
            bits_ = static_cast<uint16_t>((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);  // round to nearest even
        }
    }
    bfloat16(double d) : bfloat16(static_cast<float>(d)) {}
    bfloat16(int i) : bfloat16(static_cast<float>(i)) {}
    float to_float() const {
        const uint32_t u = static_cast<uint32_t>(bits_) << 16;
        float f;
        std::memcpy(&f, &u, 4);
        return f;
    }
    operator float() const { return to_float(); }
    uint16_t to_uint16() const { return bits_; }
    static bfloat16 from_bits(uint16_t b) {
        bfloat16 r;
        r.bits_ = b;
        return r;
    }
};
static_assert(sizeof(bfloat16) == 2, "bfloat16 must be 16 bits");

constexpr size_t DEFAULT_L1_SMALL_SIZE = 0;
constexpr size_t DEFAULT_TRACE_REGION_SIZE = 0;

namespace tt {

namespace stl {
template <typename T>
struct Span {
    T* ptr = nullptr;
    size_t len = 0;
    Span() = default;
    Span(T* p, size_t n) : ptr(p), len(n) {}
    template <typename A>
    Span(std::vector<A>& v) : ptr(v.data()), len(v.size()) {}
    template <typename A>
    Span(const std::vector<A>& v) : ptr(v.data()), len(v.size()) {}
    T* data() const { return ptr; }
    size_t size() const { return len; }
    T* begin() const { return ptr; }
    T* end() const { return ptr + len; }
    T& operator[](size_t i) const { return ptr[i]; }
};
}  // namespace stl

namespace tt_fabric {
enum class FabricConfig { DISABLED, FABRIC_1D, FABRIC_2D };
// NVLink / NVSwitch needs no fabric bring-up.
inline void SetFabricConfig(FabricConfig) {}
}  // namespace tt_fabric

namespace tt_metal {

namespace b200_detail {
[[noreturn]] inline void fail(const char* what, int code) {
    throw std::runtime_error(std::string(what) + ": " + b200_last_error() + " (status " + std::to_string(code) + ")");
}
inline void check(int code, const char* what) {
    if (code != B200_OK) fail(what, code);
}
}  // namespace b200_detail

enum class DataType { BFLOAT16 = 0, FLOAT32 = 1, UINT32 = 2 };
enum class Layout { ROW_MAJOR = 0, TILE = 1 };
enum class BufferType { DRAM, L1 };
enum class TensorMemoryLayout { INTERLEAVED };
enum class MathFidelity { LoFi = 0, HiFi2 = 2, HiFi3 = 3, HiFi4 = 4 };

struct MemoryConfig {
    TensorMemoryLayout memory_layout = TensorMemoryLayout::INTERLEAVED;
    BufferType buffer_type = BufferType::DRAM;
    MemoryConfig() = default;
    MemoryConfig(TensorMemoryLayout l, BufferType b) : memory_layout(l), buffer_type(b) {}
};

struct DispatchCoreConfig {};

struct CoreCoord {
    size_t x = 0, y = 0;
    CoreCoord() = default;
    CoreCoord(size_t x_, size_t y_) : x(x_), y(y_) {}
};
struct CoreRange {
    CoreCoord start_coord, end_coord;
    CoreRange(CoreCoord s, CoreCoord e) : start_coord(s), end_coord(e) {}
};
struct CoreRangeSet {
    std::vector<CoreRange> ranges;
    CoreRangeSet() = default;
    CoreRangeSet(const CoreRange& r) : ranges{r} {}
    CoreRangeSet(std::vector<CoreRange> r) : ranges(std::move(r)) {}
    CoreRangeSet(std::initializer_list<CoreRange> r) : ranges(r) {}
};

// Shape: rank <= 8, negative indexing, value semantics.
class Shape {
    std::vector<uint32_t> dims_;

public:
    Shape() = default;
    Shape(std::initializer_list<uint32_t> d) : dims_(d) {}
    explicit Shape(std::vector<uint32_t> d) : dims_(std::move(d)) {}
    template <size_t N>
    explicit Shape(const std::array<uint32_t, N>& d) : dims_(d.begin(), d.end()) {}
    size_t rank() const { return dims_.size(); }
    size_t size() const { return dims_.size(); }
    uint32_t operator[](int i) const {
        const int r = static_cast<int>(dims_.size());
        if (i < 0) i += r;
        if (i < 0 || i >= r) throw std::out_of_range("Shape index out of range");
        return dims_[static_cast<size_t>(i)];
    }
    uint32_t& operator[](int i) {
        const int r = static_cast<int>(dims_.size());
        if (i < 0) i += r;
        if (i < 0 || i >= r) throw std::out_of_range("Shape index out of range");
        return dims_[static_cast<size_t>(i)];
    }
    uint64_t volume() const {
        uint64_t v = 1;
        for (uint32_t d : dims_) v *= d;
        return v;
    }
    bool operator==(const Shape& o) const { return dims_ == o.dims_; }
    bool operator!=(const Shape& o) const { return dims_ != o.dims_; }
    auto begin() const { return dims_.begin(); }
    auto end() const { return dims_.end(); }
    const std::vector<uint32_t>& view() const { return dims_; }
};
inline std::ostream& operator<<(std::ostream& os, const Shape& s) {
    os << "Shape([";
    for (size_t i = 0; i < s.rank(); ++i) os << (i ? ", " : "") << s[static_cast<int>(i)];
    return os << "])";
}

struct PageConfig {
    Layout layout;
    PageConfig(Layout l = Layout::TILE) : layout(l) {}
};
struct TensorLayout {
    DataType dtype;
    PageConfig page_config;
    MemoryConfig memory_config;
    TensorLayout(DataType d, PageConfig p, MemoryConfig m = MemoryConfig{}) : dtype(d), page_config(p), memory_config(m) {}
};
struct TensorSpec {
    Shape shape;
    TensorLayout layout;
    TensorSpec(Shape s, TensorLayout l) : shape(std::move(s)), layout(l) {}
    const Shape& logical_shape() const { return shape; }
};

namespace distributed {

struct MeshShape {
    uint32_t rows = 1, cols = 1;
    MeshShape() = default;
    MeshShape(uint32_t r, uint32_t c) : rows(r), cols(c) {}
    uint32_t mesh_size() const { return rows * cols; }
};
struct MeshCoordinate {
    uint32_t row = 0, col = 0;
    MeshCoordinate(uint32_t r = 0, uint32_t c = 0) : row(r), col(c) {}
};
struct MeshDeviceConfig {
    MeshShape shape;
    explicit MeshDeviceConfig(MeshShape s = MeshShape{}) : shape(s) {}
};
struct MeshTraceId {
    uint32_t id = 0;
    uint32_t get() const { return id; }
    bool operator==(const MeshTraceId& o) const { return id == o.id; }
};
inline std::ostream& operator<<(std::ostream& os, const MeshTraceId& t) { return os << t.id; }

class MeshDevice;
struct MeshCommandQueue {
    MeshDevice* device = nullptr;
};

// One GPU per mesh position; position 0 is the device the single-device API talks to.
class MeshDevice : public std::enable_shared_from_this<MeshDevice> {
    std::vector<b200_ctx*> ctx_;
    std::vector<int> ordinals_;
    MeshShape shape_;
    std::vector<MeshCommandQueue> cqs_;
    bool open_ = false;

public:
    MeshDevice(const std::vector<int>& ordinals, MeshShape shape, int num_cqs) : ordinals_(ordinals), shape_(shape) {
        for (int ord : ordinals_) {
            b200_ctx* c = nullptr;
            b200_detail::check(b200_ctx_create(ord, &c), "MeshDevice: b200_ctx_create");
            ctx_.push_back(c);
        }
        for (size_t i = 0; i < ctx_.size(); ++i)
            for (size_t j = i + 1; j < ctx_.size(); ++j)
                b200_detail::check(b200_enable_peer_access(ctx_[i], ctx_[j]), "MeshDevice: peer access");
        cqs_.resize(static_cast<size_t>(std::max(1, num_cqs)));
        for (auto& q : cqs_) q.device = this;
        open_ = true;
    }
    ~MeshDevice() { close(); }
    MeshDevice(const MeshDevice&) = delete;
    MeshDevice& operator=(const MeshDevice&) = delete;

    static std::shared_ptr<MeshDevice> create_unit_mesh(int device_id, size_t /*l1_small_size*/ = DEFAULT_L1_SMALL_SIZE,
                                                        size_t /*trace_region_size*/ = DEFAULT_TRACE_REGION_SIZE,
                                                        int num_command_queues = 1,
                                                        const DispatchCoreConfig& = DispatchCoreConfig{}) {
        return std::make_shared<MeshDevice>(std::vector<int>{device_id}, MeshShape(1, 1), num_command_queues);
    }
    static std::shared_ptr<MeshDevice> create(const MeshDeviceConfig& cfg, size_t = DEFAULT_L1_SMALL_SIZE,
                                              size_t = DEFAULT_TRACE_REGION_SIZE, int num_command_queues = 1,
                                              const DispatchCoreConfig& = DispatchCoreConfig{}) {
        std::vector<int> ords;
        for (uint32_t i = 0; i < cfg.shape.mesh_size(); ++i) ords.push_back(static_cast<int>(i));
        return std::make_shared<MeshDevice>(ords, cfg.shape, num_command_queues);
    }

    b200_ctx* ctx(size_t i = 0) const {
        if (!open_ || i >= ctx_.size()) throw std::runtime_error("MeshDevice: device is closed or index out of range");
        return ctx_[i];
    }
    size_t num_devices() const { return ctx_.size(); }
    const MeshShape& shape() const { return shape_; }
    MeshCommandQueue& mesh_command_queue(size_t cq_id = 0) { return cqs_[std::min(cq_id, cqs_.size() - 1)]; }
    // The Tensix worker grid has no counterpart; report the SM count as a 1-row grid.
    CoreCoord compute_with_storage_grid_size() const {
        int sms = 0;
        b200_detail::check(b200_ctx_sm_count(ctx(0), &sms), "b200_ctx_sm_count");
        return CoreCoord(static_cast<size_t>(sms), 1);
    }
    void synchronize() {
        for (b200_ctx* c : ctx_) b200_detail::check(b200_synchronize(c, nullptr), "Synchronize");
    }
    // Every device's stream waits for the work queued so far on every other device's stream (events, no host wait):
    // what a device runs next then sees whatever its peers stored into its memory.
    void order_all_streams() {
        for (size_t i = 0; i < ctx_.size(); ++i)
            for (size_t j = 0; j < ctx_.size(); ++j)
                if (i != j) b200_detail::check(b200_ctx_wait_ctx(ctx_[i], ctx_[j]), "MeshDevice: stream order");
    }

    bool close() {
        if (!open_) return false;
        open_ = false;
        for (b200_ctx* c : ctx_) b200_ctx_destroy(c);
        ctx_.clear();
        return true;
    }
    bool is_open() const { return open_; }
};

inline void Finish(MeshCommandQueue& cq) { cq.device->synchronize(); }
template <typename Opt = std::nullopt_t>
inline void Synchronize(MeshDevice* dev, Opt = std::nullopt) {
    dev->synchronize();
}

}  // namespace distributed

// ---------------------------------------------------------------------------------------------------------------------
// Tensor
// ---------------------------------------------------------------------------------------------------------------------
namespace b200_detail {

inline size_t dtype_size(DataType d) { return d == DataType::BFLOAT16 ? 2 : 4; }
inline int abi_dtype(DataType d) { return d == DataType::BFLOAT16 ? B200_BF16 : (d == DataType::FLOAT32 ? B200_F32 : B200_U32); }

struct Storage {
    distributed::MeshDevice* device = nullptr;  // nullptr: host tensor
    size_t device_index = 0;
    void* dptr = nullptr;
    std::vector<uint8_t> host;
    size_t bytes = 0;
    std::shared_ptr<distributed::MeshDevice> keep_alive;

    Storage() = default;
    Storage(const Storage&) = delete;
    Storage& operator=(const Storage&) = delete;
    ~Storage() { release(); }
    void release() {
        if (dptr && device && device->is_open()) b200_pool_free(device->ctx(device_index), dptr);
        dptr = nullptr;
    }
};

inline std::shared_ptr<Storage> device_storage(distributed::MeshDevice* dev, size_t bytes, size_t index = 0) {
    auto st = std::make_shared<Storage>();
    st->device = dev;
    st->device_index = index;
    st->bytes = bytes;
    check(b200_pool_alloc(dev->ctx(index), std::max<size_t>(bytes, 16), &st->dptr), "tensor allocation");
    return st;
}

}  // namespace b200_detail

class Tensor {
    std::shared_ptr<b200_detail::Storage> st_;
    // Mesh tensors (one shard per device of a multi-device mesh) keep the extra shards here; st_ is shard 0.
    std::vector<std::shared_ptr<b200_detail::Storage>> shards_;
    Shape shape_;
    DataType dtype_ = DataType::BFLOAT16;
    Layout layout_ = Layout::TILE;

public:
    Tensor() = default;
    Tensor(std::shared_ptr<b200_detail::Storage> st, Shape shape, DataType dtype, Layout layout)
        : st_(std::move(st)), shape_(std::move(shape)), dtype_(dtype), layout_(layout) {}

    const Shape& logical_shape() const { return shape_; }
    const Shape& padded_shape() const { return shape_; }
    const Shape& shape() const { return shape_; }
    DataType dtype() const { return dtype_; }
    Layout layout() const { return layout_; }
    uint64_t volume() const { return shape_.volume(); }
    uint64_t physical_volume() const { return shape_.volume(); }
    bool is_allocated() const { return st_ != nullptr && (st_->dptr != nullptr || !st_->host.empty() || st_->bytes == 0); }
    bool on_device() const { return st_ && st_->device != nullptr; }
    distributed::MeshDevice* device() const { return st_ ? st_->device : nullptr; }
    size_t device_index() const { return st_ ? st_->device_index : 0; }
    void* device_ptr() const { return st_ ? st_->dptr : nullptr; }
    const std::shared_ptr<b200_detail::Storage>& storage() const { return st_; }
    // Mesh tensors: one storage per device of the mesh, all with this tensor's (per-device) shape.
    const std::vector<std::shared_ptr<b200_detail::Storage>>& shards() const { return shards_; }
    size_t num_shards() const { return shards_.empty() ? 1 : shards_.size(); }
    Tensor shard(size_t i) const {
        if (shards_.empty()) return *this;
        return Tensor(shards_.at(i), shape_, dtype_, layout_);
    }
    static Tensor from_shards(const std::vector<Tensor>& parts) {
        Tensor t = parts.at(0);
        if (parts.size() > 1) {
            t.shards_.clear();
            for (const Tensor& p : parts) t.shards_.push_back(p.st_);
        }
        return t;
    }
    MemoryConfig memory_config() const { return MemoryConfig{}; }

    // Same storage, different shape (ttnn::reshape is a view here: storage is always contiguous row-major).
    Tensor view(Shape s, Layout l) const {
        if (s.volume() != shape_.volume()) throw std::invalid_argument("reshape: element count differs");
        Tensor t(st_, std::move(s), dtype_, l);
        return t;
    }
    Tensor with_layout(Layout l) const { return Tensor(st_, shape_, dtype_, l); }

    void deallocate(bool /*force*/ = false) {
        if (st_ && st_.use_count() == 1) st_->release();
        st_.reset();
        shards_.clear();
    }

    // Host <-> device --------------------------------------------------------------------------------------------
    template <typename T>
    static Tensor from_vector(const std::vector<T>& v, const TensorSpec& spec, distributed::MeshDevice* device = nullptr) {
        if (v.size() != spec.shape.volume()) throw std::invalid_argument("from_vector: size does not match the shape");
        auto st = std::make_shared<b200_detail::Storage>();
        const DataType dt = spec.layout.dtype;
        st->bytes = v.size() * b200_detail::dtype_size(dt);
        st->host.resize(st->bytes);
        if (dt == DataType::BFLOAT16) {
            auto* out = reinterpret_cast<uint16_t*>(st->host.data());
            for (size_t i = 0; i < v.size(); ++i) {
                if constexpr (std::is_same_v<T, bfloat16>)
                    out[i] = v[i].to_uint16();
                else
                    out[i] = bfloat16(static_cast<float>(v[i])).to_uint16();
            }
        } else if (dt == DataType::FLOAT32) {
            auto* out = reinterpret_cast<float*>(st->host.data());
            for (size_t i = 0; i < v.size(); ++i) out[i] = static_cast<float>(v[i]);
        } else {
            auto* out = reinterpret_cast<uint32_t*>(st->host.data());
            for (size_t i = 0; i < v.size(); ++i) out[i] = static_cast<uint32_t>(static_cast<float>(v[i]));
        }
        Tensor t(st, spec.shape, dt, spec.layout.page_config.layout);
        return device ? t.to_device(device) : t;
    }

    Tensor to_device(distributed::MeshDevice* dev, const MemoryConfig& = MemoryConfig{}, size_t index = 0) const {
        if (!st_) throw std::runtime_error("to_device: empty tensor");
        if (on_device()) return *this;
        auto st = b200_detail::device_storage(dev, st_->bytes, index);
        if (st_->bytes)
            b200_detail::check(b200_memcpy_h2d(dev->ctx(index), st->dptr, st_->host.data(), st_->bytes, nullptr), "to_device");
        // the host bytes may be freed by the caller right after this returns
        b200_detail::check(b200_synchronize(dev->ctx(index), nullptr), "to_device");
        return Tensor(st, shape_, dtype_, layout_);
    }

    Tensor cpu(bool /*blocking*/ = true) const {
        if (!st_) throw std::runtime_error("cpu: empty tensor");
        if (!on_device()) return *this;
        auto st = std::make_shared<b200_detail::Storage>();
        st->bytes = st_->bytes;
        st->host.resize(st_->bytes);
        if (st_->bytes)
            b200_detail::check(b200_memcpy_d2h(st_->device->ctx(st_->device_index), st->host.data(), st_->dptr, st_->bytes,
                                               nullptr), "Tensor::cpu");
        return Tensor(st, shape_, dtype_, layout_);
    }

    template <typename T>
    std::vector<T> to_vector() const {
        const Tensor h = on_device() ? cpu() : *this;
        const size_t n = static_cast<size_t>(shape_.volume());
        std::vector<T> out(n);
        const uint8_t* p = h.st_->host.data();
        for (size_t i = 0; i < n; ++i) {
            float f;
            if (dtype_ == DataType::BFLOAT16)
                f = bfloat16::from_bits(reinterpret_cast<const uint16_t*>(p)[i]).to_float();
            else if (dtype_ == DataType::FLOAT32)
                f = reinterpret_cast<const float*>(p)[i];
            else
                f = static_cast<float>(reinterpret_cast<const uint32_t*>(p)[i]);
            if constexpr (std::is_same_v<T, bfloat16>)
                out[i] = bfloat16(f);
            else
                out[i] = static_cast<T>(f);
        }
        return out;
    }
};

inline std::ostream& operator<<(std::ostream& os, const Tensor& t) {
    return os << "Tensor(" << t.logical_shape() << (t.on_device() ? ", device)" : ", host)");
}

}  // namespace tt_metal
}  // namespace tt

// ---------------------------------------------------------------------------------------------------------------------
// ttnn: names and operations
// ---------------------------------------------------------------------------------------------------------------------
using MathFidelity = tt::tt_metal::MathFidelity;  // the reference uses the enum unqualified (verify/verify_fidelity.cpp:23)

namespace ttnn {

using tt::tt_metal::BufferType;
using tt::tt_metal::CoreCoord;
using tt::tt_metal::CoreRange;
using tt::tt_metal::CoreRangeSet;
using tt::tt_metal::DataType;
using tt::tt_metal::Layout;
using tt::tt_metal::MemoryConfig;
using tt::tt_metal::PageConfig;
using tt::tt_metal::Shape;
using tt::tt_metal::Tensor;
using tt::tt_metal::TensorLayout;
using tt::tt_metal::TensorMemoryLayout;
using tt::tt_metal::TensorSpec;
using MeshDevice = tt::tt_metal::distributed::MeshDevice;
using ::bfloat16;

constexpr Layout TILE_LAYOUT = Layout::TILE;
constexpr Layout ROW_MAJOR_LAYOUT = Layout::ROW_MAJOR;
const MemoryConfig DRAM_MEMORY_CONFIG{TensorMemoryLayout::INTERLEAVED, BufferType::DRAM};
const MemoryConfig L1_MEMORY_CONFIG{TensorMemoryLayout::INTERLEAVED, BufferType::L1};

struct CoreGrid {
    size_t x = 0, y = 0;
    CoreGrid() = default;
    CoreGrid(size_t x_, size_t y_) : x(x_), y(y_) {}
};

// WormholeComputeKernelConfig{math_fidelity, math_approx_mode, fp32_dest_acc_en, packer_l1_acc} (verify_fidelity.cpp:50-55)
struct WormholeComputeKernelConfig {
    MathFidelity math_fidelity = MathFidelity::HiFi4;
    bool math_approx_mode = false;
    bool fp32_dest_acc_en = false;
    bool packer_l1_acc = false;
    bool dst_full_sync_en = false;
};
using DeviceComputeKernelConfig = WormholeComputeKernelConfig;

namespace operations {
namespace matmul {
struct MatmulProgramConfig {};
}  // namespace matmul
namespace unary {
enum class UnaryOpType { RELU, GELU };
struct EltwiseUnaryWithParam {
    UnaryOpType op_type;
    EltwiseUnaryWithParam(UnaryOpType t) : op_type(t) {}
};
using UnaryWithParam = EltwiseUnaryWithParam;
}  // namespace unary
}  // namespace operations

namespace detail {

using tt::tt_metal::b200_detail::abi_dtype;
using tt::tt_metal::b200_detail::check;
using tt::tt_metal::b200_detail::device_storage;
using tt::tt_metal::b200_detail::dtype_size;

inline MeshDevice* dev_of(const Tensor& t, const char* op) {
    if (!t.on_device()) throw std::runtime_error(std::string(op) + ": tensor is not on a device");
    return t.device();
}
inline b200_ctx* ctx_of(const Tensor& t, const char* op) { return dev_of(t, op)->ctx(t.device_index()); }

inline Tensor alloc_like(const Tensor& ref, Shape shape, DataType dt, Layout layout, const char* op) {
    MeshDevice* dev = dev_of(ref, op);
    auto st = device_storage(dev, shape.volume() * dtype_size(dt), ref.device_index());
    return Tensor(st, std::move(shape), dt, layout);
}
inline Tensor alloc_on(MeshDevice& dev, Shape shape, DataType dt, Layout layout) {
    auto st = device_storage(&dev, shape.volume() * dtype_size(dt), 0);
    return Tensor(st, std::move(shape), dt, layout);
}

inline void shape4(const Shape& s, int64_t (&out)[4], const char* op) {
    if (s.rank() > 4) throw std::invalid_argument(std::string(op) + ": rank > 4 is not supported");
    for (int i = 0; i < 4; ++i) out[i] = 1;
    for (size_t i = 0; i < s.rank(); ++i) out[4 - s.rank() + i] = s[static_cast<int>(i)];
}

inline Shape broadcast_shape(const Shape& a, const Shape& b, const char* op) {
    const size_t r = std::max(a.rank(), b.rank());
    std::vector<uint32_t> out(r, 1);
    for (size_t i = 0; i < r; ++i) {
        const uint32_t da = i < r - a.rank() ? 1 : a[static_cast<int>(i - (r - a.rank()))];
        const uint32_t db = i < r - b.rank() ? 1 : b[static_cast<int>(i - (r - b.rank()))];
        if (da != db && da != 1 && db != 1) throw std::invalid_argument(std::string(op) + ": shapes do not broadcast");
        out[i] = std::max(da, db);
    }
    return Shape(out);
}

// Runs a single-device op on every device of a mesh tensor and reassembles the results.
template <typename Fn>
inline Tensor per_shard(const Tensor& a, Fn&& fn) {
    if (a.num_shards() == 1) return fn(a, 0);
    std::vector<Tensor> parts;
    for (size_t i = 0; i < a.num_shards(); ++i) parts.push_back(fn(a.shard(i), i));
    return Tensor::from_shards(parts);
}

inline Tensor binary1(int op, const Tensor& a, const Tensor& b, const char* name);
inline Tensor binary(int op, const Tensor& a, const Tensor& b, const char* name) {
    return per_shard(a, [&](const Tensor& as, size_t i) { return binary1(op, as, b.shard(i), name); });
}
inline Tensor binary1(int op, const Tensor& a, const Tensor& b, const char* name) {
    const Shape os = broadcast_shape(a.logical_shape(), b.logical_shape(), name);
    Tensor out = alloc_like(a, os, DataType::BFLOAT16, a.layout(), name);
    int64_t sa[4], sb[4];
    shape4(a.logical_shape(), sa, name);
    shape4(b.logical_shape(), sb, name);
    check(b200_binary(ctx_of(a, name), op, a.device_ptr(), sa, b.device_ptr(), sb, out.device_ptr(), nullptr), name);
    return out;
}
inline Tensor unary1(int op, const Tensor& x, float scalar, const char* name);
inline Tensor unary(int op, const Tensor& x, float scalar, const char* name) {
    return per_shard(x, [&](const Tensor& xs, size_t) { return unary1(op, xs, scalar, name); });
}
inline Tensor unary1(int op, const Tensor& x, float scalar, const char* name) {
    Tensor out = alloc_like(x, x.logical_shape(), DataType::BFLOAT16, x.layout(), name);
    check(b200_unary(ctx_of(x, name), op, x.device_ptr(), out.device_ptr(), static_cast<int64_t>(x.volume()), scalar, nullptr),
          name);
    return out;
}

inline int fidelity_of(const std::optional<DeviceComputeKernelConfig>& cfg) {
    if (!cfg) return B200_HIFI4;
    switch (cfg->math_fidelity) {
        case MathFidelity::LoFi: return B200_LOFI;
        case MathFidelity::HiFi2: return B200_HIFI2;
        case MathFidelity::HiFi3: return B200_HIFI3;
        default: return B200_HIFI4;
    }
}
inline int activation_of(const std::optional<std::string>& act) {
    if (!act || act->empty()) return B200_ACT_NONE;
    if (*act == "relu") return B200_ACT_RELU;
    if (*act == "gelu") return B200_ACT_GELU;
    throw std::invalid_argument("unsupported fused activation '" + *act + "'");
}

inline Tensor matmul_impl(const Tensor& a, const Tensor& b, bool ta, bool tb, const Tensor* bias,
                          const std::optional<std::string>& activation,
                          const std::optional<DeviceComputeKernelConfig>& cfg, const char* name) {
    const Shape& as = a.logical_shape();
    const Shape& bs = b.logical_shape();
    if (as.rank() < 2 || bs.rank() < 2) throw std::invalid_argument(std::string(name) + ": operands must have rank >= 2");
    const uint32_t am = ta ? as[-1] : as[-2], ak = ta ? as[-2] : as[-1];
    const uint32_t bk = tb ? bs[-1] : bs[-2], bn = tb ? bs[-2] : bs[-1];
    if (ak != bk) throw std::invalid_argument(std::string(name) + ": inner dimensions differ");
    uint64_t batch_a = 1, batch_b = 1;
    for (size_t i = 0; i + 2 < as.rank(); ++i) batch_a *= as[static_cast<int>(i)];
    for (size_t i = 0; i + 2 < bs.rank(); ++i) batch_b *= bs[static_cast<int>(i)];
    std::vector<uint32_t> od(as.view().begin(), as.view().end());
    od[od.size() - 2] = am;
    od[od.size() - 1] = bn;
    b200_gemm_desc d;
    b200_gemm_desc_init(&d);
    d.transpose_a = ta;
    d.transpose_b = tb;
    d.K = ak;
    d.N = bn;
    d.A = a.device_ptr();
    d.B = b.device_ptr();
    d.lda = as[-1];
    d.ldb = bs[-1];
    d.ldc = bn;
    if (batch_b == 1 && !ta) {  // [.., M, K] x [K, N]: one product over all leading positions
        d.M = static_cast<int64_t>(batch_a) * am;
        d.batch = 1;
    } else {
        if (batch_b != 1 && batch_b != batch_a) throw std::invalid_argument(std::string(name) + ": batch dimensions differ");
        d.M = am;
        d.batch = static_cast<int64_t>(batch_a);
        d.stride_a = static_cast<int64_t>(as[-2]) * as[-1];
        d.stride_b = batch_b == 1 ? 0 : static_cast<int64_t>(bs[-2]) * bs[-1];
        d.stride_c = static_cast<int64_t>(am) * bn;
    }
    Tensor out = alloc_like(a, Shape(od), (cfg && cfg->fp32_dest_acc_en && false) ? DataType::FLOAT32 : DataType::BFLOAT16,
                            a.layout(), name);
    d.C = out.device_ptr();
    if (bias) {
        if (bias->logical_shape()[-1] != bn || bias->volume() != bn)
            throw std::invalid_argument(std::string(name) + ": bias must be a [1, N] row");
        d.bias = bias->device_ptr();
    }
    d.activation = activation_of(activation);
    d.fidelity = fidelity_of(cfg);
    check(b200_gemm(ctx_of(a, name), &d, nullptr), name);
    return out;
}

// [outer, R, inner] view of `dim` of shape s
inline void reduce_view(const Shape& s, int dim, int64_t& outer, int64_t& R, int64_t& inner) {
    const int r = static_cast<int>(s.rank());
    if (dim < 0) dim += r;
    if (dim < 0 || dim >= r) throw std::out_of_range("reduction dim out of range");
    outer = inner = 1;
    for (int i = 0; i < dim; ++i) outer *= s[i];
    R = s[dim];
    for (int i = dim + 1; i < r; ++i) inner *= s[i];
}

inline Tensor reduce(int op, const Tensor& x, std::optional<int> dim, bool keepdim, const char* name) {
    const Shape& s = x.logical_shape();
    int64_t outer, R, inner;
    std::vector<uint32_t> od;
    if (dim) {
        reduce_view(s, *dim, outer, R, inner);
        int dd = *dim < 0 ? *dim + static_cast<int>(s.rank()) : *dim;
        for (int i = 0; i < static_cast<int>(s.rank()); ++i) {
            if (i == dd) {
                if (keepdim) od.push_back(1);
            } else {
                od.push_back(s[i]);
            }
        }
    } else {
        outer = 1;
        R = static_cast<int64_t>(s.volume());
        inner = 1;
        if (keepdim) od.assign(s.rank(), 1);
    }
    if (od.empty()) od.push_back(1);
    Tensor out = alloc_like(x, Shape(od), DataType::BFLOAT16, x.layout(), name);
    check(b200_reduce(ctx_of(x, name), op, x.device_ptr(), outer, R, inner, out.device_ptr(), nullptr), name);
    return out;
}

inline Tensor filled(const Shape& shape, float value, DataType dt, Layout layout, MeshDevice& dev) {
    std::vector<Tensor> parts;  // on a multi-device mesh the tensor is replicated on every device
    for (size_t i = 0; i < dev.num_devices(); ++i) {
        auto st = device_storage(&dev, shape.volume() * dtype_size(dt), i);
        Tensor out(st, shape, dt, layout);
        check(b200_fill(dev.ctx(i), out.device_ptr(), static_cast<int64_t>(shape.volume()), abi_dtype(dt), value, nullptr),
              "fill");
        parts.push_back(out);
    }
    return Tensor::from_shards(parts);
}

}  // namespace detail

// ---- matmul / linear (dynamic/ops.hpp:21-46, static/nn.hpp:145-146, bench/metal/bench_fusion.cpp:83,119,
//      verify/verify_fidelity.cpp:66-67, traced/mesh.hpp:142-144: positional optionals) ------------------------------
inline Tensor matmul(const Tensor& a, const Tensor& b, bool transpose_a = false, bool transpose_b = false,
                     const std::optional<MemoryConfig>& = std::nullopt, const std::optional<DataType>& = std::nullopt,
                     const std::optional<operations::matmul::MatmulProgramConfig>& = std::nullopt,
                     const std::optional<std::string>& activation = std::nullopt,
                     const std::optional<DeviceComputeKernelConfig>& compute_kernel_config = std::nullopt,
                     const std::optional<CoreGrid>& = std::nullopt) {
    return detail::per_shard(a, [&](const Tensor& as, size_t i) {
        return detail::matmul_impl(as, b.shard(i), transpose_a, transpose_b, nullptr, activation, compute_kernel_config,
                                   "ttnn::matmul");
    });
}

inline Tensor linear(const Tensor& a, const Tensor& w, const std::optional<Tensor>& bias = std::nullopt,
                     bool transpose_a = false, bool transpose_b = false, const std::optional<MemoryConfig>& = std::nullopt,
                     const std::optional<DataType>& = std::nullopt,
                     const std::optional<operations::matmul::MatmulProgramConfig>& = std::nullopt,
                     const std::optional<std::string>& activation = std::nullopt,
                     const std::optional<DeviceComputeKernelConfig>& compute_kernel_config = std::nullopt,
                     const std::optional<CoreGrid>& = std::nullopt) {
    return detail::matmul_impl(a, w, transpose_a, transpose_b, bias ? &*bias : nullptr, activation, compute_kernel_config,
                               "ttnn::linear");
}

// ---- element-wise -------------------------------------------------------------------------------------------------
inline Tensor add(const Tensor& a, const Tensor& b) { return detail::binary(B200_B_ADD, a, b, "ttnn::add"); }
inline Tensor subtract(const Tensor& a, const Tensor& b) { return detail::binary(B200_B_SUB, a, b, "ttnn::subtract"); }
inline Tensor multiply(const Tensor& a, const Tensor& b) { return detail::binary(B200_B_MUL, a, b, "ttnn::multiply"); }
inline Tensor divide(const Tensor& a, const Tensor& b) { return detail::binary(B200_B_DIV, a, b, "ttnn::divide"); }
inline Tensor add(const Tensor& a, float s) { return detail::unary(B200_U_ADD_SCALAR, a, s, "ttnn::add"); }
inline Tensor subtract(const Tensor& a, float s) { return detail::unary(B200_U_ADD_SCALAR, a, -s, "ttnn::subtract"); }
inline Tensor multiply(const Tensor& a, float s) { return detail::unary(B200_U_MUL_SCALAR, a, s, "ttnn::multiply"); }
inline Tensor divide(const Tensor& a, float s) { return detail::unary(B200_U_MUL_SCALAR, a, 1.0f / s, "ttnn::divide"); }

#define B200_TTNN_UNARY(fn, op)                                                                                         \
    inline Tensor fn(const Tensor& x, const std::optional<MemoryConfig>& = std::nullopt,                                \
                     const std::optional<Tensor>& = std::nullopt, const std::optional<CoreRangeSet>& = std::nullopt) { \
        return detail::unary(op, x, 0.0f, "ttnn::" #fn);                                                               \
    }
B200_TTNN_UNARY(neg, B200_U_NEG)
B200_TTNN_UNARY(relu, B200_U_RELU)
B200_TTNN_UNARY(gtz, B200_U_GTZ)
B200_TTNN_UNARY(rsqrt, B200_U_RSQRT)
B200_TTNN_UNARY(exp, B200_U_EXP)
B200_TTNN_UNARY(log, B200_U_LOG)
B200_TTNN_UNARY(tanh, B200_U_TANH)
B200_TTNN_UNARY(sqrt, B200_U_SQRT)
B200_TTNN_UNARY(reciprocal, B200_U_RECIP)
B200_TTNN_UNARY(square, B200_U_SQUARE)
#undef B200_TTNN_UNARY
inline Tensor gelu(const Tensor& x, bool /*fast_and_approximate_mode*/ = false) {
    return detail::unary(B200_U_GELU, x, 0.0f, "ttnn::gelu");
}

// ttnn::gelu_bw(dy, x, "none") -> {dx} (traced/ops.hpp:96-99)
inline std::vector<std::optional<Tensor>> gelu_bw(const Tensor& dy, const Tensor& x, const std::string& /*approximate*/ = "none") {
    return {detail::binary(B200_B_GELU_BW, dy, x, "ttnn::gelu_bw")};
}
inline std::vector<std::optional<Tensor>> relu_bw(const Tensor& dy, const Tensor& x) {
    return {detail::binary(B200_B_RELU_BW, dy, x, "ttnn::relu_bw")};
}

inline Tensor triu(const Tensor& x, int diagonal = 0) {
    const Shape& s = x.logical_shape();
    Tensor out = detail::alloc_like(x, s, DataType::BFLOAT16, x.layout(), "ttnn::triu");
    const int64_t rows = s[-2], cols = s[-1];
    detail::check(b200_triu(detail::ctx_of(x, "ttnn::triu"), x.device_ptr(), out.device_ptr(),
                            static_cast<int64_t>(s.volume()) / (rows * cols), rows, cols, diagonal, nullptr), "ttnn::triu");
    return out;
}

// ---- reductions / softmax -----------------------------------------------------------------------------------------
inline Tensor sum(const Tensor& x, std::optional<int> dim = std::nullopt, bool keepdim = false) {
    return detail::reduce(B200_R_SUM, x, dim, keepdim, "ttnn::sum");
}
inline Tensor mean(const Tensor& x, std::optional<int> dim = std::nullopt, bool keepdim = false) {
    return detail::reduce(B200_R_MEAN, x, dim, keepdim, "ttnn::mean");
}
inline Tensor max(const Tensor& x, std::optional<int> dim = std::nullopt, bool keepdim = false) {
    return detail::reduce(B200_R_MAX, x, dim, keepdim, "ttnn::max");
}

inline Tensor softmax(const Tensor& x, int dim = -1, const std::optional<MemoryConfig>& = std::nullopt,
                      const std::optional<DeviceComputeKernelConfig>& = std::nullopt) {
    const Shape& s = x.logical_shape();
    const int r = static_cast<int>(s.rank());
    if (dim < 0) dim += r;
    if (dim != r - 1) throw std::invalid_argument("ttnn::softmax: only the last dimension is supported");
    Tensor out = detail::alloc_like(x, s, DataType::BFLOAT16, x.layout(), "ttnn::softmax");
    const int64_t cols = s[-1], rows = static_cast<int64_t>(s.volume()) / std::max<int64_t>(cols, 1);
    detail::check(b200_softmax(detail::ctx_of(x, "ttnn::softmax"), x.device_ptr(), cols, out.device_ptr(), cols, rows, cols,
                               1.0f, 0, nullptr), "ttnn::softmax");
    return out;
}

// ---- fused attention --------------------------------------------------------------------------------------------------
// ttnn::transformer::scaled_dot_product_attention on [B, H, S, 64] tensors: softmax(scale * Q K^T [+ causal mask]) V in one
// kernel (b200_attention_forward), without the [S, S] score tensor that the matmul / softmax / matmul composition of
// autograd/traced/nn.hpp:164-175 writes. The reference's executors do not call it; it is offered for code that does.
namespace transformer {
inline Tensor scaled_dot_product_attention(const Tensor& q, const Tensor& k, const Tensor& v,
                                           const std::optional<Tensor>& attn_mask = std::nullopt, bool is_causal = true,
                                           std::optional<float> scale = std::nullopt) {
    const char* op = "ttnn::transformer::scaled_dot_product_attention";
    if (attn_mask) throw std::invalid_argument(std::string(op) + ": explicit masks are not supported, use is_causal");
    const Shape& s = q.logical_shape();
    if (s.rank() != 4 || k.logical_shape() != s || v.logical_shape() != s)
        throw std::invalid_argument(std::string(op) + ": q, k, v must share one [B, H, S, dh] shape");
    const int64_t B = s[0], H = s[1], S = s[2], dh = s[3];
    Tensor out = detail::alloc_like(q, s, DataType::BFLOAT16, q.layout(), op);
    auto lse = detail::device_storage(detail::dev_of(q, op), static_cast<size_t>(B * H * S) * sizeof(float), q.device_index());
    auto operand = [&](const Tensor& t) { return b200_attn_operand{const_cast<void*>(t.device_ptr()), H * S * dh, S * dh, dh}; };
    const b200_attn_operand qo = operand(q), ko = operand(k), vo = operand(v), oo = operand(out);
    detail::check(b200_attention_forward(detail::ctx_of(q, op), &qo, &ko, &vo, &oo, static_cast<float*>(lse->dptr), B, H, S,
                                         static_cast<int>(dh), scale.value_or(1.0f / std::sqrt(static_cast<float>(dh))),
                                         is_causal ? 1 : 0, nullptr),
                  op);
    return out;
}
}  // namespace transformer

// ---- layout ---------------------------------------------------------------------------------------------------------
inline Tensor reshape(const Tensor& x, const Shape& shape) { return x.view(shape, x.layout()); }
inline Tensor untilize(const Tensor& x) { return x.with_layout(Layout::ROW_MAJOR); }
inline Tensor tilize(const Tensor& x) { return x.with_layout(Layout::TILE); }
inline Tensor to_layout(const Tensor& x, Layout l) { return x.with_layout(l); }

inline Tensor transpose(const Tensor& x, int d0, int d1) {
    const Shape& s = x.logical_shape();
    const int r = static_cast<int>(s.rank());
    if (d0 < 0) d0 += r;
    if (d1 < 0) d1 += r;
    if (d0 < 0 || d1 < 0 || d0 >= r || d1 >= r || r > 4) throw std::out_of_range("ttnn::transpose: bad dims");
    int64_t in4[4];
    detail::shape4(s, in4, "ttnn::transpose");
    int32_t perm[4] = {0, 1, 2, 3};
    std::swap(perm[4 - r + d0], perm[4 - r + d1]);
    std::vector<uint32_t> od(s.view());
    std::swap(od[static_cast<size_t>(d0)], od[static_cast<size_t>(d1)]);
    Tensor out = detail::alloc_like(x, Shape(od), x.dtype(), x.layout(), "ttnn::transpose");
    detail::check(b200_permute(detail::ctx_of(x, "ttnn::transpose"), x.device_ptr(), in4, perm, out.device_ptr(), nullptr),
                  "ttnn::transpose");
    return out;
}

// ---- embedding (traced/nn.hpp:303-315) ---------------------------------------------------------------------------
inline Tensor embedding(const Tensor& indices, const Tensor& weight, const std::optional<int>& /*pad_token*/ = std::nullopt,
                        const Layout& layout = Layout::ROW_MAJOR) {
    const Shape& ws = weight.logical_shape();
    const int64_t vocab = ws[-2], dim = ws[-1], n = static_cast<int64_t>(indices.volume());
    std::vector<uint32_t> od(indices.logical_shape().view());
    od.push_back(static_cast<uint32_t>(dim));
    Tensor out = detail::alloc_like(weight, Shape(od), DataType::BFLOAT16, layout, "ttnn::embedding");
    detail::check(b200_embedding_forward(detail::ctx_of(weight, "ttnn::embedding"),
                                         static_cast<const uint32_t*>(indices.device_ptr()), n, weight.device_ptr(), vocab, dim,
                                         out.device_ptr(), nullptr), "ttnn::embedding");
    return out;
}

// d_out is [1, 1, B*S, D]; the result has the weight's shape (as ttnn::embedding_bw: [1, 1, vocab, dim]).
inline Tensor embedding_bw(const Tensor& indices, const Tensor& weight, const Tensor& d_out,
                           const std::optional<DataType>& = std::nullopt) {
    const Shape& ws = weight.logical_shape();
    const int64_t vocab = ws[-2], dim = ws[-1], n = static_cast<int64_t>(indices.volume());
    b200_ctx* ctx = detail::ctx_of(weight, "ttnn::embedding_bw");
    Tensor acc = detail::alloc_like(weight, ws, DataType::FLOAT32, weight.layout(), "ttnn::embedding_bw");
    detail::check(b200_embedding_backward(ctx, static_cast<const uint32_t*>(indices.device_ptr()), n, d_out.device_ptr(), vocab,
                                          dim, static_cast<float*>(acc.device_ptr()), nullptr), "ttnn::embedding_bw");
    Tensor out = detail::alloc_like(weight, Shape({1, 1, static_cast<uint32_t>(vocab), static_cast<uint32_t>(dim)}),
                                    DataType::BFLOAT16, Layout::TILE, "ttnn::embedding_bw");
    detail::check(b200_cast(ctx, acc.device_ptr(), B200_F32, out.device_ptr(), B200_BF16, vocab * dim, nullptr),
                  "ttnn::embedding_bw");
    return out;
}

// ---- creation -------------------------------------------------------------------------------------------------------
inline Tensor full(const Shape& shape, float value, DataType dt, Layout layout, MeshDevice& dev,
                   const std::optional<MemoryConfig>& = std::nullopt) {
    return detail::filled(shape, value, dt, layout, dev);
}
inline Tensor zeros(const Shape& shape, DataType dt, Layout layout, MeshDevice& dev,
                    const std::optional<MemoryConfig>& = std::nullopt) {
    return detail::filled(shape, 0.0f, dt, layout, dev);
}
inline Tensor ones(const Shape& shape, DataType dt, Layout layout, MeshDevice& dev,
                   const std::optional<MemoryConfig>& = std::nullopt) {
    return detail::filled(shape, 1.0f, dt, layout, dev);
}
inline Tensor full_like(const Tensor& t, float value) {
    Tensor out = detail::alloc_like(t, t.logical_shape(), t.dtype(), t.layout(), "ttnn::full_like");
    detail::check(b200_fill(detail::ctx_of(t, "ttnn::full_like"), out.device_ptr(), static_cast<int64_t>(t.volume()),
                            detail::abi_dtype(t.dtype()), value, nullptr), "ttnn::full_like");
    return out;
}
inline Tensor zeros_like(const Tensor& t) { return full_like(t, 0.0f); }
inline Tensor ones_like(const Tensor& t) { return full_like(t, 1.0f); }

namespace random {
// Host tensor of uniform bf16 values (dynamic/autograd.hpp:99).
inline Tensor uniform(bfloat16 low, bfloat16 high, const Shape& shape, Layout layout = Layout::TILE, uint32_t seed = 0) {
    static std::mt19937 fallback_engine(5489u);
    std::mt19937 seeded(seed);
    std::mt19937& eng = seed ? seeded : fallback_engine;
    std::uniform_real_distribution<float> dist(low.to_float(), high.to_float());
    std::vector<bfloat16> v(static_cast<size_t>(shape.volume()));
    for (auto& x : v) x = bfloat16(dist(eng));
    return Tensor::from_vector(v, TensorSpec(shape, TensorLayout(DataType::BFLOAT16, PageConfig(layout), MemoryConfig{})));
}
}  // namespace random

inline Tensor to_device(const Tensor& t, MeshDevice* dev, const std::optional<MemoryConfig>& = std::nullopt) {
    return t.to_device(dev);
}
inline Tensor from_device(const Tensor& t) { return t.cpu(); }

// ---- device ---------------------------------------------------------------------------------------------------------
inline std::shared_ptr<MeshDevice> open_mesh_device(int device_id, size_t l1_small = DEFAULT_L1_SMALL_SIZE,
                                                    size_t trace_region = DEFAULT_TRACE_REGION_SIZE, int num_cqs = 1) {
    return MeshDevice::create_unit_mesh(device_id, l1_small, trace_region, num_cqs);
}
inline void close_device(MeshDevice& dev) { dev.close(); }
inline void close_mesh_device(const std::shared_ptr<MeshDevice>& dev) {
    if (dev) dev->close();
}

// ---- mesh tensors: mappers, distribute_tensor, all_gather (bench/metal/matmul_tensor_parallel.cpp:70-92, :153-186) ---
namespace distributed {
using tt::tt_metal::distributed::MeshShape;

struct TensorToMesh {
    MeshDevice* mesh = nullptr;
    int shard_dim = -1;  // -1: replicate
};

inline std::unique_ptr<TensorToMesh> replicate_tensor_to_mesh_mapper(MeshDevice& mesh) {
    return std::make_unique<TensorToMesh>(TensorToMesh{&mesh, -1});
}
inline std::unique_ptr<TensorToMesh> shard_tensor_to_mesh_mapper(MeshDevice& mesh, int dim) {
    return std::make_unique<TensorToMesh>(TensorToMesh{&mesh, dim});
}

// Host tensor -> one shard (or replica) per device of the mesh. Slicing happens on the host, as in the reference.
inline Tensor distribute_tensor(const Tensor& host, const TensorToMesh& mapper,
                                std::optional<std::reference_wrapper<MeshDevice>> mesh = std::nullopt) {
    MeshDevice& dev = mesh ? mesh->get() : *mapper.mesh;
    const size_t n = dev.num_devices();
    const Tensor h = host.on_device() ? host.cpu() : host;
    const Shape& s = h.logical_shape();
    const size_t es = detail::dtype_size(h.dtype());
    std::vector<Tensor> parts;
    if (mapper.shard_dim < 0) {
        for (size_t i = 0; i < n; ++i) parts.push_back(h.to_device(&dev, MemoryConfig{}, i));
        return Tensor::from_shards(parts);
    }
    int dim = mapper.shard_dim < 0 ? mapper.shard_dim + static_cast<int>(s.rank()) : mapper.shard_dim;
    if (dim >= static_cast<int>(s.rank()) || s[dim] % n != 0)
        throw std::invalid_argument("shard_tensor_to_mesh_mapper: dimension is not divisible by the mesh size");
    uint64_t outer = 1, inner = 1;
    for (int i = 0; i < dim; ++i) outer *= s[i];
    for (int i = dim + 1; i < static_cast<int>(s.rank()); ++i) inner *= s[i];
    const uint64_t piece = s[dim] / n;
    std::vector<uint32_t> sd(s.view());
    sd[static_cast<size_t>(dim)] = static_cast<uint32_t>(piece);
    const uint8_t* src = h.storage()->host.data();
    for (size_t i = 0; i < n; ++i) {
        auto st = std::make_shared<tt::tt_metal::b200_detail::Storage>();
        st->bytes = outer * piece * inner * es;
        st->host.resize(st->bytes);
        for (uint64_t o = 0; o < outer; ++o)
            std::memcpy(st->host.data() + o * piece * inner * es, src + (o * s[dim] + i * piece) * inner * es, piece * inner * es);
        parts.push_back(Tensor(st, Shape(sd), h.dtype(), h.layout()).to_device(&dev, MemoryConfig{}, i));
    }
    return Tensor::from_shards(parts);
}

inline std::shared_ptr<MeshDevice> open_mesh_device(const MeshShape& shape, size_t l1_small = DEFAULT_L1_SMALL_SIZE,
                                                    size_t trace_region = DEFAULT_TRACE_REGION_SIZE, int num_cqs = 1,
                                                    const tt::tt_metal::DispatchCoreConfig& cfg = {}) {
    return MeshDevice::create(tt::tt_metal::distributed::MeshDeviceConfig(shape), l1_small, trace_region, num_cqs, cfg);
}
inline void close_mesh_device(const std::shared_ptr<MeshDevice>& dev) {
    if (dev) dev->close();
}
}  // namespace distributed

// Every device ends with the concatenation of all devices' shards along `dim` (copy engines over NVLink, ordered after
// the producing ops). The fused form — matmul whose epilogue stores into every peer — is b200_gemm_allgather.
inline Tensor all_gather(const Tensor& t, int dim, int /*num_links*/ = 1) {
    const size_t n = t.num_shards();
    if (n == 1) return t;
    const Shape& s = t.logical_shape();
    if (dim < 0) dim += static_cast<int>(s.rank());
    uint64_t outer = 1, inner = 1;
    for (int i = 0; i < dim; ++i) outer *= s[i];
    for (int i = dim; i < static_cast<int>(s.rank()); ++i) inner *= s[i];  // contiguous run of one shard per outer index
    const size_t es = detail::dtype_size(t.dtype());
    std::vector<uint32_t> od(s.view());
    od[static_cast<size_t>(dim)] *= static_cast<uint32_t>(n);
    MeshDevice* dev = t.device();
    std::vector<Tensor> parts;
    for (size_t d = 0; d < n; ++d) {
        auto st = detail::device_storage(dev, Shape(od).volume() * es, d);
        Tensor out(st, Shape(od), t.dtype(), t.layout());
        for (size_t src = 0; src < n; ++src) {
            const Tensor sh = t.shard(src);
            detail::check(b200_peer_copy_2d(dev->ctx(d), static_cast<uint8_t*>(out.device_ptr()) + src * inner * es,
                                            n * inner * es, dev->ctx(src), sh.device_ptr(), inner * es, inner * es, outer),
                          "ttnn::all_gather");
        }
        parts.push_back(out);
    }
    return Tensor::from_shards(parts);
}

// The inverse exchange (no signature exists in the reference; the K-split matmul of the distributed configuration
// needs it): every device holds a full-shape partial result; afterwards device d holds the sum over all devices of
// slice d along `dim`. Unfused form: slices travel by copy engine, the sum runs in fp32 on the owner. The fused form
// — a matmul whose epilogue stores its fp32 partial tiles straight into the owner's memory — is
// ttnn::experimental::matmul_reduce_scatter below.
inline Tensor reduce_scatter(const Tensor& t, int dim, int /*num_links*/ = 1) {
    const size_t n = t.num_shards();
    if (n == 1) return t;
    const Shape& s = t.logical_shape();
    if (dim < 0) dim += static_cast<int>(s.rank());
    if (dim < 0 || dim >= static_cast<int>(s.rank()) || s[dim] % n != 0)
        throw std::invalid_argument("ttnn::reduce_scatter: dimension is not divisible by the mesh size");
    if (t.dtype() != DataType::BFLOAT16) throw std::invalid_argument("ttnn::reduce_scatter: bfloat16 tensors only");
    uint64_t outer = 1, inner = 1;
    for (int i = 0; i < dim; ++i) outer *= s[i];
    for (int i = dim + 1; i < static_cast<int>(s.rank()); ++i) inner *= s[i];
    const uint64_t piece = s[dim] / n;                       // slice length along dim
    const size_t es = detail::dtype_size(t.dtype());
    const uint64_t run = piece * inner;                      // contiguous elements of one slice per outer index
    std::vector<uint32_t> od(s.view());
    od[static_cast<size_t>(dim)] = static_cast<uint32_t>(piece);
    MeshDevice* dev = t.device();
    std::vector<Tensor> parts;
    for (size_t d = 0; d < n; ++d) {
        // staging [n][outer][run] on the owner, then one column sum over the n copies
        auto stage = detail::device_storage(dev, n * outer * run * es, d);
        for (size_t src = 0; src < n; ++src) {
            const Tensor sh = t.shard(src);
            detail::check(b200_peer_copy_2d(dev->ctx(d), static_cast<uint8_t*>(stage->dptr) + src * outer * run * es, run * es,
                                            dev->ctx(src), static_cast<const uint8_t*>(sh.device_ptr()) + d * run * es,
                                            n * run * es, run * es, outer),
                          "ttnn::reduce_scatter");
        }
        auto st = detail::device_storage(dev, outer * run * es, d);
        Tensor out(st, Shape(od), t.dtype(), t.layout());
        detail::check(b200_reduce(dev->ctx(d), B200_R_SUM, stage->dptr, 1, static_cast<int64_t>(n),
                                  static_cast<int64_t>(outer * run), out.device_ptr(), nullptr),
                      "ttnn::reduce_scatter");
        parts.push_back(out);
    }
    return Tensor::from_shards(parts);
}

namespace experimental {

// C = A . B on a mesh with A replicated and B sharded on its columns (shard_tensor_to_mesh_mapper(mesh, 1)), every
// device ending with the whole C: ttnn::matmul followed by ttnn::all_gather(c, 1) of
// bench/metal/matmul_tensor_parallel.cpp:84-92 as ONE op per device. The GEMM epilogue stores each finished tile into
// every device's C over NVLink while the tensor cores work on the next tiles (b200_gemm_allgather); no gather pass runs.
inline Tensor matmul_all_gather(const Tensor& a, const Tensor& b) {
    const size_t n = b.num_shards();
    MeshDevice* dev = a.device();
    if (n == 1) return matmul(a, b);
    if (a.num_shards() != n) throw std::invalid_argument("matmul_all_gather: A must be replicated on the mesh of B");
    const Shape& as = a.logical_shape();
    const Shape& bs = b.logical_shape();
    if (as.rank() != 2 || bs.rank() != 2 || as[1] != bs[0]) throw std::invalid_argument("matmul_all_gather: [M,K] x [K,N/n] operands");
    const uint32_t M = as[0], K = as[1], Ns = bs[1];
    std::vector<Tensor> outs;
    std::vector<void*> peer_c;
    for (size_t d = 0; d < n; ++d) {
        auto st = detail::device_storage(dev, static_cast<size_t>(M) * Ns * n * 2, d);
        outs.emplace_back(st, Shape({M, static_cast<uint32_t>(Ns * n)}), DataType::BFLOAT16, a.layout());
        peer_c.push_back(outs.back().device_ptr());
    }
    for (size_t d = 0; d < n; ++d) {
        b200_gemm_desc g;
        b200_gemm_desc_init(&g);
        g.M = M; g.N = Ns; g.K = K;
        g.A = a.shard(d).device_ptr(); g.lda = K;
        g.B = b.shard(d).device_ptr(); g.ldb = Ns;
        g.ldc = static_cast<int64_t>(Ns) * n;
        detail::check(b200_gemm_allgather(dev->ctx(d), &g, peer_c.data(), static_cast<int>(n), static_cast<int>(d), nullptr),
                      "matmul_all_gather");
    }
    dev->order_all_streams();   // a device's later ops see the tiles its peers stored into its C
    return Tensor::from_shards(outs);
}

// C = A . B with A sharded on its columns and B on its rows (both on K): device d ends with row block d of C. The
// fp32 partial tiles go from the GEMM epilogue straight into the owner's staging slots; each owner then sums its n
// slots and rounds to bf16 once (b200_gemm_reduce_scatter_partials + b200_reduce_slices). The staging blocks go back
// to their pool when this function returns; that is safe because a pooled block is only ever reused by later work on
// the owner's stream, which is ordered after the sum, which is ordered after every peer's stores.
inline Tensor matmul_reduce_scatter(const Tensor& a, const Tensor& b) {
    const size_t n = a.num_shards();
    MeshDevice* dev = a.device();
    if (n == 1) return matmul(a, b);
    if (b.num_shards() != n) throw std::invalid_argument("matmul_reduce_scatter: A and B must be sharded on the same mesh");
    const Shape& as = a.logical_shape();
    const Shape& bs = b.logical_shape();
    if (as.rank() != 2 || bs.rank() != 2 || as[1] != bs[0]) throw std::invalid_argument("matmul_reduce_scatter: [M,K/n] x [K/n,N] operands");
    const uint32_t M = as[0], Ks = as[1], N = bs[1];
    if (M % n != 0) throw std::invalid_argument("matmul_reduce_scatter: M is not divisible by the mesh size");
    const uint32_t rows = M / static_cast<uint32_t>(n);
    std::vector<std::shared_ptr<tt::tt_metal::b200_detail::Storage>> slots;
    std::vector<void*> peer_slots;
    for (size_t d = 0; d < n; ++d) {
        slots.push_back(detail::device_storage(dev, n * static_cast<size_t>(rows) * N * 4, d));
        peer_slots.push_back(slots.back()->dptr);
    }
    for (size_t d = 0; d < n; ++d) {
        b200_gemm_desc g;
        b200_gemm_desc_init(&g);
        g.M = M; g.N = N; g.K = Ks;
        g.A = a.shard(d).device_ptr(); g.lda = Ks;
        g.B = b.shard(d).device_ptr(); g.ldb = N;
        g.ldc = N;
        g.c_dtype = B200_F32;
        detail::check(b200_gemm_reduce_scatter_partials(dev->ctx(d), &g, peer_slots.data(), static_cast<int>(n),
                                                        static_cast<int>(d), nullptr),
                      "matmul_reduce_scatter");
    }
    dev->order_all_streams();
    std::vector<Tensor> outs;
    for (size_t d = 0; d < n; ++d) {
        auto st = detail::device_storage(dev, static_cast<size_t>(rows) * N * 2, d);
        outs.emplace_back(st, Shape({rows, N}), DataType::BFLOAT16, a.layout());
        b200_gemm_desc g;
        b200_gemm_desc_init(&g);
        g.M = rows; g.N = N; g.K = 0;
        g.C = outs.back().device_ptr(); g.ldc = N;
        detail::check(b200_reduce_slices(dev->ctx(d), static_cast<const float*>(slots[d]->dptr), static_cast<int>(n), &g, nullptr),
                      "matmul_reduce_scatter");
    }
    return Tensor::from_shards(outs);
}

}  // namespace experimental

// ---- softmax cross-entropy (the reference has it only in Python: CrossEntropyLoss, py/nn.py:149-222; torch form
//      experiment_torch.py:183). logits [rows, classes] bf16, labels [rows] uint32 class ids on the device.
//      loss: fp32 [1, 1], the mean over rows; d_logits: (softmax - onehot) / rows in bf16 — one fused pass, no one-hot
//      tensor (the Python reference builds it on the host each step, py/nn.py:180-188). --------------------------------
struct CrossEntropyResult {
    Tensor loss;
    Tensor d_logits;
};
inline CrossEntropyResult cross_entropy(const Tensor& logits, const Tensor& labels) {
    const Shape& s = logits.logical_shape();
    if (s.rank() < 2 || logits.dtype() != DataType::BFLOAT16) throw std::invalid_argument("ttnn::cross_entropy: bf16 [rows, classes] logits");
    const int64_t classes = s[-1];
    const int64_t rows = static_cast<int64_t>(s.volume()) / classes;
    if (labels.dtype() != DataType::UINT32 || static_cast<int64_t>(labels.volume()) != rows)
        throw std::invalid_argument("ttnn::cross_entropy: labels must be one uint32 class id per row");
    CrossEntropyResult r{detail::alloc_like(logits, Shape({1, 1}), DataType::FLOAT32, logits.layout(), "ttnn::cross_entropy"),
                         detail::alloc_like(logits, s, DataType::BFLOAT16, logits.layout(), "ttnn::cross_entropy")};
    b200_ctx* c = detail::ctx_of(logits, "ttnn::cross_entropy");
    detail::check(b200_memset(c, r.loss.device_ptr(), 0, 4, nullptr), "ttnn::cross_entropy");
    detail::check(b200_cross_entropy(c, logits.device_ptr(), classes, static_cast<const uint32_t*>(labels.device_ptr()), rows,
                                     classes, 1.0f / static_cast<float>(rows), static_cast<float*>(r.loss.device_ptr()), nullptr,
                                     r.d_logits.device_ptr(), classes, nullptr),
                  "ttnn::cross_entropy");
    return r;
}

// ---- traces (traced/trace.hpp:57-78) ----------------------------------------------------------------------------------
namespace operations {
namespace trace {
using MeshTraceId = tt::tt_metal::distributed::MeshTraceId;
template <typename Cq = std::nullopt_t>
inline MeshTraceId begin_trace_capture(MeshDevice* dev, Cq = std::nullopt) {
    MeshTraceId id;
    detail::check(b200_trace_begin(dev->ctx(0), &id.id), "begin_trace_capture");
    return id;
}
template <typename Cq = std::nullopt_t>
inline void end_trace_capture(MeshDevice* dev, MeshTraceId id, Cq = std::nullopt) {
    detail::check(b200_trace_end(dev->ctx(0), id.id), "end_trace_capture");
}
template <typename Cq = std::nullopt_t>
inline void execute_trace(MeshDevice* dev, MeshTraceId id, Cq = std::nullopt, bool blocking = false) {
    detail::check(b200_trace_execute(dev->ctx(0), id.id, blocking ? 1 : 0), "execute_trace");
}
inline void release_trace(MeshDevice* dev, MeshTraceId id) {
    if (dev && dev->is_open()) detail::check(b200_trace_release(dev->ctx(0), id.id), "release_trace");
}
}  // namespace trace
}  // namespace operations

}  // namespace ttnn
