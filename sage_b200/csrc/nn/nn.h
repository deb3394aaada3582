// Layers and the two workload graphs.  Reference: src/layers.rs (Dense :208-247, Conv2d :327-404,
// Embedding :406-463, LayerNorm :548-590, Softmax :249-273, MaxPool2d :56-88, AdaptiveAvgPool2d
// :124-154, Flatten :198-206, Sequential :275-325), src/models/bert.rs, src/models/resnet.rs.
#pragma once
#include <memory>
#include <vector>

#include "../graph/graph.h"

namespace sage {
namespace nn {

struct Layer {
    virtual ~Layer() {}
    virtual Var pass(const Var &x) const = 0;
    virtual void params(std::vector<Var> *p) const {}
    virtual void buffers(std::vector<Var> *p) const {}  // state that is not a parameter (BatchNorm2d's running statistics)
};

struct Dense : Layer {
    Var weight, bias;
    Dense(long long din, long long dout);
    Var pass(const Var &x) const override;
    void params(std::vector<Var> *p) const override;
};

struct Conv2d : Layer {
    Var weight, bias;
    ops::Pair stride, pad, dil;
    Conv2d(long long cin, long long cout, ops::Pair ker, ops::Pair stride, ops::Pair pad, ops::Pair dil);
    Var pass(const Var &x) const override;
    void params(std::vector<Var> *p) const override;
};

struct Embedding : Layer {
    long long dim;
    Var weight;
    Embedding(long long n, long long dim);
    Var pass(const Var &idx) const override;
    void params(std::vector<Var> *p) const override;
};

struct LayerNorm : Layer {
    std::vector<long long> axes;
    float eps;
    Var gamma, beta;
    LayerNorm(const std::vector<long long> &axes, float eps);
    Var pass(const Var &x) const override;
    void params(std::vector<Var> *p) const override;
};

// layers.rs:479-546: inference-mode normalisation with running statistics per channel; gamma / beta are [1]
// tensors; the layer always passes eps = 1e-05 (layers.rs:542) whatever it was constructed with.
// Only gamma and beta are parameters (layers.rs:528-531); the running statistics are `buffers`.
struct BatchNorm2d : Layer {
    float eps;
    Var gamma, beta, running_mean, running_var;
    BatchNorm2d(long long num_features, float eps);
    Var pass(const Var &x) const override;
    void params(std::vector<Var> *p) const override;
    void buffers(std::vector<Var> *p) const override;
};

struct Softmax : Layer {  // layers.rs:249-273
    long long axis;
    explicit Softmax(long long a) : axis(a) {}
    Var pass(const Var &x) const override { return ops::softmax(x, {axis}); }
};
struct Relu : Layer {
    Var pass(const Var &x) const override { return ops::relu(x); }
};
struct Gelu : Layer {  // not in the reference: 0.5 x (1 + erf(x / sqrt 2)) from the reference's map ops
    Var pass(const Var &x) const override;
};
struct MaxPool2d : Layer {
    ops::Pair ker, stride, pad, dil;
    MaxPool2d(ops::Pair k, ops::Pair s, ops::Pair p, ops::Pair d) : ker(k), stride(s), pad(p), dil(d) {}
    Var pass(const Var &x) const override { return ops::max_pool_2d(x, ker, stride, pad, dil); }
};
struct AvgPool2d : Layer {  // layers.rs:90-122
    ops::Pair ker, stride, pad, dil;
    AvgPool2d(ops::Pair k, ops::Pair s, ops::Pair p, ops::Pair d) : ker(k), stride(s), pad(p), dil(d) {}
    Var pass(const Var &x) const override { return ops::avg_pool_2d(x, ker, stride, pad, dil); }
};
struct AdaptiveAvgPool2d : Layer {
    ops::Pair ext;
    explicit AdaptiveAvgPool2d(ops::Pair e) : ext(e) {}
    Var pass(const Var &x) const override;
};
struct Flatten : Layer {
    Var pass(const Var &x) const override { return ops::view(x, {x.extent(0), -1}); }
};
struct Sequential : Layer {
    std::vector<std::shared_ptr<Layer>> layers;
    Sequential &add(std::shared_ptr<Layer> l) {
        layers.push_back(std::move(l));
        return *this;
    }
    Var pass(const Var &x) const override;
    void params(std::vector<Var> *p) const override;
    void buffers(std::vector<Var> *p) const override;
};

// models/bert.rs:8-55.  `base()` is the reference's constructor; the other fields let the harness
// build the BERT-large-shaped and GELU / eps variants that the reference's private config cannot.
struct BertConfig {
    long long embed_dim = 768, num_vocabs = 30522, max_num_tokens = 512, hidden_dim = 3072, num_layers = 12,
              num_heads = 12, num_classes = 2;
    int gelu = 0;             // 0: ReLU feed-forward like the reference (bert.rs:190-194)
    float layer_norm_eps = 1e-05f;  // the reference's LayerNorm::pass hard-codes 1e-05 (layers.rs:586-589)
};

struct MultiHeadAttention {
    long long num_heads, head_dim;
    Dense key_proj, query_proj, value_proj, dense;
    LayerNorm norm;
    explicit MultiHeadAttention(const BertConfig &c);
    Var pass(const Var &x, const Var &mask) const;
    void params(std::vector<Var> *p) const;
};

struct BertLayer {
    MultiHeadAttention attention;
    Sequential ffn;
    LayerNorm norm;
    explicit BertLayer(const BertConfig &c);
    Var pass(const Var &x, const Var &mask) const;
    void params(std::vector<Var> *p) const;
};

struct Bert {
    Embedding word_emb, pos_emb;
    LayerNorm emb_norm;
    std::vector<std::unique_ptr<BertLayer>> layers;
    Dense classifier;
    explicit Bert(const BertConfig &c);
    Var pass(const Var &token_ids, const Var &mask) const;  // bert.rs:72-81
    void params(std::vector<Var> *p) const;                 // bert.rs:90-94 traversal order
};

// models/resnet.rs:74-129 with ResNetConfig::d18.  BatchNorm is commented out in the reference (:80, :167, :170);
// `batch_norm` puts a BatchNorm2d back at exactly those three places (after the first convolution and after
// both convolutions of every BasicLayer), which is the inference-BatchNorm variant of the workload.
std::shared_ptr<Sequential> resnet18(long long chan_input, long long num_classes, bool batch_norm = false);
// models/densenet.rs:56-107: DenseNetConfig::d121 / d169 / d201 are (depth, growth rate) = (121, 12), (169, 24), (201, 12);
// BatchNorm and dropout are declared in the reference's config but never applied.
std::shared_ptr<Sequential> densenet(long long chan_input, long long num_classes, long long depth, long long growth_rate);
// models/mobilenet.rs:38-80 with MobileNetV2Config::new (width multiplier 1).
std::shared_ptr<Sequential> mobilenet_v2(long long chan_in, long long num_classes);

}  // namespace nn
}  // namespace sage
