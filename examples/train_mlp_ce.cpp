// MLP training with softmax cross-entropy on the reference's dynamic autograd executor.
//
// The reference's examples/train_mlp.cpp trains Linear -> ReLU -> Linear with an MSE loss (and no longer compiles
// against its own headers: it re-defines `MLP` and `mse_loss`, which dynamic/nn.hpp and dynamic/ops.hpp now provide).
// The MNIST-shaped configuration of this repository's benchmarks needs the same loop with integer labels and a
// cross-entropy loss, which the reference only has in Python (py/nn.py:149-222). This program is that loop: the
// reference's executor headers (dynamic/autograd.hpp, ops.hpp, nn.hpp, optim.hpp) are used UNCHANGED; the only
// addition is one autograd node, `cross_entropy`, on top of ttnn::cross_entropy of the stand-in TTNN.
//
//   train_mlp_ce                       batch 64, 784 -> 128 -> 10, uniform(-0.1, 0.1) weights, random data, lr 0.01
//   train_mlp_ce <dir>                 reads x.bin [64,784] f32, labels.bin [64] u32, w1.bin [128,784], b1.bin [128],
//                                      w2.bin [10,128], b2.bin [10] (f32) from <dir>: a seeded case whose loss
//                                      trajectory a test compares with the CPU oracle
// Prints one line per step: "step <i> loss <fp32 mean loss>".
#include "dynamic/autograd.hpp"
#include "dynamic/ops.hpp"
#include "dynamic/nn.hpp"
#include "dynamic/optim.hpp"
#include "common.hpp"

#include <cstdio>
#include <fstream>
#include <iostream>
#include <random>
#include <string>
#include <vector>

using namespace autograd;

// loss = mean_rows( -log softmax(logits)[label] ); d_logits = (softmax - onehot) / rows, both from one fused pass.
// The loss Value holds an fp32 [1, 1] tensor; its backward hands the stored d_logits to the logits node (the upstream
// gradient of a loss is 1, which is what autograd::backward seeds).
inline ValuePtr cross_entropy(ValuePtr logits, const tt::tt_metal::Tensor& labels) {
    auto r = ttnn::cross_entropy(logits->data, labels);
    auto out = std::make_shared<Value>(r.loss, logits->requires_grad, "cross_entropy", std::vector<ValuePtr>{logits});
    auto d_logits = r.d_logits;
    out->backward_fn = [logits, d_logits]() { logits->accumulate_grad(d_logits); };
    return out;
}

template <typename T>
static std::vector<T> read_bin(const std::string& path, size_t count) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot open " + path);
    std::vector<T> v(count);
    f.read(reinterpret_cast<char*>(v.data()), static_cast<std::streamsize>(count * sizeof(T)));
    if (static_cast<size_t>(f.gcount()) != count * sizeof(T)) throw std::runtime_error(path + " is too short");
    return v;
}

static tt::tt_metal::Tensor upload_bf16(const std::vector<float>& v, ttnn::Shape shape, MeshDevice& device) {
    std::vector<bfloat16> h(v.begin(), v.end());
    auto spec = tt::tt_metal::TensorSpec(shape, tt::tt_metal::TensorLayout(DataType::BFLOAT16,
                                                                          tt::tt_metal::PageConfig(Layout::TILE), MemoryConfig{}));
    return tt::tt_metal::Tensor::from_vector(h, spec).to_device(&device);
}

int main(int argc, char** argv) {
    test::DeviceGuard dg;
    auto& device = dg.get();
    const uint32_t batch = 64, in_features = 784, hidden = 128, classes = 10;
    const float lr = 0.01f;
    const int steps = 10;

    MLP model(in_features, hidden, classes, device);
    std::vector<float> xs(batch * in_features);
    std::vector<uint32_t> ys(batch);
    if (argc > 1) {
        const std::string dir = argv[1];
        xs = read_bin<float>(dir + "/x.bin", xs.size());
        ys = read_bin<uint32_t>(dir + "/labels.bin", ys.size());
        model.layer1.weight->data = upload_bf16(read_bin<float>(dir + "/w1.bin", hidden * in_features), ttnn::Shape({hidden, in_features}), device);
        model.layer1.bias->data = upload_bf16(read_bin<float>(dir + "/b1.bin", hidden), ttnn::Shape({1, hidden}), device);
        model.layer2.weight->data = upload_bf16(read_bin<float>(dir + "/w2.bin", classes * hidden), ttnn::Shape({classes, hidden}), device);
        model.layer2.bias->data = upload_bf16(read_bin<float>(dir + "/b2.bin", classes), ttnn::Shape({1, classes}), device);
    } else {
        std::mt19937 gen(42);
        std::normal_distribution<float> nd(0.0f, 1.0f);
        std::uniform_int_distribution<uint32_t> ud(0, classes - 1);
        for (auto& v : xs) v = nd(gen);
        for (auto& v : ys) v = ud(gen);
    }
    auto x = from_tensor(upload_bf16(xs, ttnn::Shape({batch, in_features}), device), false, "input");
    auto label_spec = tt::tt_metal::TensorSpec(ttnn::Shape({batch}), tt::tt_metal::TensorLayout(DataType::UINT32,
                                               tt::tt_metal::PageConfig(Layout::ROW_MAJOR), MemoryConfig{}));
    auto labels = tt::tt_metal::Tensor::from_vector(ys, label_spec).to_device(&device);

    SGD sgd(model.parameters(), lr);
    float first = 0.0f, last = 0.0f;
    for (int i = 0; i < steps; ++i) {
        sgd.zero_grad();
        auto logits = model.forward(x);
        auto loss = cross_entropy(logits, labels);
        backward(loss, device);
        sgd.step();
        Finish(device.mesh_command_queue());
        const float v = loss->data.cpu().to_vector<float>()[0];
        std::printf("step %d loss %.6f\n", i, v);
        if (i == 0) first = v;
        last = v;
    }
    std::printf("loss reduced: %s\n", last < first ? "YES" : "NO");
    return last < first ? 0 : 1;
}
