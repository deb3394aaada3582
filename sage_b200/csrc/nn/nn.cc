#include "nn.h"

#include <cmath>

namespace sage {
namespace nn {
using namespace ops;

Dense::Dense(long long din, long long dout) : weight(Var::empty({din, dout}, SAGE_F32)), bias(Var::empty({dout}, SAGE_F32)) {
    weight.origin->name = "dense.weight";
    bias.origin->name = "dense.bias";
}
Var Dense::pass(const Var &x) const { return add(matmul(x, weight), bias); }  // layers.rs:243-247
void Dense::params(std::vector<Var> *p) const {
    p->push_back(weight);
    p->push_back(bias);
}

// layers.rs:352-365: the weight is [kernel_size.at(1), kernel_size.at(0), C, OC] = [KH, KW, C, OC]
Conv2d::Conv2d(long long cin, long long cout, Pair ker, Pair s, Pair p, Pair d)
    : weight(Var::empty({ker.h, ker.w, cin, cout}, SAGE_F32)), bias(Var::empty({cout}, SAGE_F32)), stride(s), pad(p), dil(d) {
    weight.origin->name = "conv2d.weight";
    bias.origin->name = "conv2d.bias";
}
Var Conv2d::pass(const Var &x) const { return add(conv_2d(x, weight, stride, pad, dil), bias); }
void Conv2d::params(std::vector<Var> *p) const {
    p->push_back(weight);
    p->push_back(bias);
}

Embedding::Embedding(long long n, long long d) : dim(d), weight(Var::empty({n, d}, SAGE_F32)) { weight.origin->name = "embedding.weight"; }
Var Embedding::pass(const Var &idx) const {  // layers.rs:427-452
    if (idx.rank() > 1) {
        const long long b = idx.extent(0), l = idx.extent(1);
        Var i = expand(view(idx, {b * l, 1}), {b * l, dim});
        return view(gather(weight, i, 0), {b, l, dim});
    }
    const long long l = idx.extent(0);
    Var i = expand(view(idx, {l, 1}), {l, dim});
    return view(gather(weight, i, 0), {l, dim});
}
void Embedding::params(std::vector<Var> *p) const { p->push_back(weight); }

LayerNorm::LayerNorm(const std::vector<long long> &a, float e)
    : axes(a), eps(e), gamma(Var::empty({1}, SAGE_F32)), beta(Var::empty({1}, SAGE_F32)) {
    gamma.origin->name = "layer_norm.gamma";
    beta.origin->name = "layer_norm.beta";
}
Var LayerNorm::pass(const Var &x) const { return layer_norm(x, axes, gamma, beta, eps); }
void LayerNorm::params(std::vector<Var> *p) const {
    p->push_back(gamma);
    p->push_back(beta);
}

BatchNorm2d::BatchNorm2d(long long n, float e)
    : eps(e), gamma(Var::empty({1}, SAGE_F32)), beta(Var::empty({1}, SAGE_F32)), running_mean(Var::empty({n}, SAGE_F32)),
      running_var(Var::empty({n}, SAGE_F32)) {
    gamma.origin->name = "batch_norm_2d.gamma";
    beta.origin->name = "batch_norm_2d.beta";
    running_mean.origin->name = "batch_norm_2d.running_mean";
    running_var.origin->name = "batch_norm_2d.running_var";
}
Var BatchNorm2d::pass(const Var &x) const { return batch_norm_2d(x, gamma, beta, running_mean, running_var, 1e-05f); }  // layers.rs:535-545
void BatchNorm2d::params(std::vector<Var> *p) const {
    p->push_back(gamma);
    p->push_back(beta);
}
void BatchNorm2d::buffers(std::vector<Var> *p) const {
    p->push_back(running_mean);
    p->push_back(running_var);
}

Var Gelu::pass(const Var &x) const {
    Var e = unary_map(div(x, std::sqrt(2.0f)), Erf);
    return mul(mul(x, 0.5f), add(e, 1.0f));
}

Var AdaptiveAvgPool2d::pass(const Var &x) const {  // layers.rs:141-153
    const long long iw = x.extent(2), ih = x.extent(1), ow = ext.w, oh = ext.h;
    Pair stride{iw / ow, ih / oh};
    Pair ker{iw - (ow - 1) * stride.w, ih - (oh - 1) * stride.h};
    return avg_pool_2d(x, ker, stride, Pair{0, 0}, Pair{1, 1});
}

Var Sequential::pass(const Var &x0) const {
    Var x = x0;
    for (auto &l : layers) x = l->pass(x);
    return x;
}
void Sequential::params(std::vector<Var> *p) const {
    for (auto &l : layers) l->params(p);
}
void Sequential::buffers(std::vector<Var> *p) const {
    for (auto &l : layers) l->buffers(p);
}

// ---------------------------------------------------------------- Bert (models/bert.rs)
MultiHeadAttention::MultiHeadAttention(const BertConfig &c)
    : num_heads(c.num_heads), head_dim(c.embed_dim / c.num_heads), key_proj(c.embed_dim, c.embed_dim),
      query_proj(c.embed_dim, c.embed_dim), value_proj(c.embed_dim, c.embed_dim), dense(c.embed_dim, c.embed_dim),
      norm({2}, c.layer_norm_eps) {}

Var MultiHeadAttention::pass(const Var &x, const Var &mask) const {  // bert.rs:250-314
    auto separate_heads = [&](const Var &f) { return transpose(view(f, {f.extent(0), f.extent(1), num_heads, head_dim}), 2, 1); };
    Var query = separate_heads(query_proj.pass(x));
    Var key = separate_heads(key_proj.pass(x));
    Var value = separate_heads(value_proj.pass(x));
    Var attention = div(matmul_batched(query, transpose(key, -1, -2)), std::sqrt((float)head_dim));
    Var ext_mask = mul(add(neg(view(mask, {mask.extent(0), 1, 1, mask.extent(1)})), 1.0f), -1e5f);  // extend_mask
    attention = softmax(add(attention, ext_mask), {3});
    Var av = transpose(matmul_batched(attention, value), 2, 1);  // merge_heads
    av = view(av, {av.extent(0), av.extent(1), num_heads * head_dim});
    return norm.pass(add(dense.pass(av), x));
}
void MultiHeadAttention::params(std::vector<Var> *p) const {  // bert.rs:325-331
    key_proj.params(p);
    query_proj.params(p);
    value_proj.params(p);
    dense.params(p);
    norm.params(p);
}

BertLayer::BertLayer(const BertConfig &c) : attention(c), norm({2}, c.layer_norm_eps) {
    ffn.add(std::make_shared<Dense>(c.embed_dim, c.hidden_dim));
    if (c.gelu) ffn.add(std::make_shared<Gelu>());
    else ffn.add(std::make_shared<Relu>());
    ffn.add(std::make_shared<Dense>(c.hidden_dim, c.embed_dim));
}
Var BertLayer::pass(const Var &x, const Var &mask) const {  // bert.rs:199-203
    Var interim = attention.pass(x, mask);
    return norm.pass(add(ffn.pass(interim), interim));
}
void BertLayer::params(std::vector<Var> *p) const {
    attention.params(p);
    ffn.params(p);
    norm.params(p);
}

Bert::Bert(const BertConfig &c)
    : word_emb(c.num_vocabs, c.embed_dim), pos_emb(c.max_num_tokens, c.embed_dim), emb_norm({2}, c.layer_norm_eps),
      classifier(c.embed_dim, c.num_classes) {
    for (long long i = 0; i < c.num_layers; ++i) layers.emplace_back(new BertLayer(c));
}
Var Bert::pass(const Var &token_ids, const Var &mask) const {
    // BertEmbedding::pass, bert.rs:128-139: position ids are built on the host
    const long long seq_len = token_ids.extent(1);
    std::vector<uint32_t> pos((size_t)seq_len);
    for (long long i = 0; i < seq_len; ++i) pos[(size_t)i] = (uint32_t)i;
    Var pos_ids = Var::from_tensor(Tensor::from_host({seq_len}, SAGE_U32, pos.data()));
    Var x = emb_norm.pass(add(word_emb.pass(token_ids), pos_emb.pass(pos_ids)));
    for (auto &l : layers) x = l->pass(x, mask);
    Var cls = squeeze(slice(x, 1, 1, 2), 1);  // features.index(1, 1).squeeze(1), bert.rs:76
    return classifier.pass(cls);
}
void Bert::params(std::vector<Var> *p) const {
    word_emb.params(p);
    pos_emb.params(p);
    emb_norm.params(p);
    for (auto &l : layers) l->params(p);
    classifier.params(p);
}

// ---------------------------------------------------------------- ResNet (models/resnet.rs)
struct BasicLayer : Layer {  // resnet.rs:150-177, 270-279
    Sequential main;
    std::shared_ptr<Sequential> down;
    BasicLayer(long long cin, long long planes, long long stride, bool batch_norm) {
        auto P = [](long long v) { return Pair{v, v}; };
        main.add(std::make_shared<Conv2d>(cin, planes, P(3), P(stride), P(1), P(1)));
        if (batch_norm) main.add(std::make_shared<BatchNorm2d>(planes, 1e-05f));  // resnet.rs:167
        main.add(std::make_shared<Relu>());
        main.add(std::make_shared<Conv2d>(planes, planes, P(3), P(1), P(1), P(1)));
        if (batch_norm) main.add(std::make_shared<BatchNorm2d>(planes, 1e-05f));  // resnet.rs:170
        if (stride != 1 || cin != planes) {
            down = std::make_shared<Sequential>();
            down->add(std::make_shared<Conv2d>(cin, planes, P(1), P(stride), P(0), P(1)));
        }
    }
    Var pass(const Var &x) const override {
        Var y = main.pass(x);
        return relu(add(y, down ? down->pass(x) : x));
    }
    void params(std::vector<Var> *p) const override {
        main.params(p);
        if (down) down->params(p);
    }
    void buffers(std::vector<Var> *p) const override {
        main.buffers(p);
        if (down) down->buffers(p);
    }
};

std::shared_ptr<Sequential> resnet18(long long chan_input, long long num_classes, bool batch_norm) {
    auto P = [](long long v) { return Pair{v, v}; };
    auto m = std::make_shared<Sequential>();
    m->add(std::make_shared<Conv2d>(chan_input, 64, P(7), P(2), P(3), P(1)));
    if (batch_norm) m->add(std::make_shared<BatchNorm2d>(64, 1e-05f));  // resnet.rs:80
    m->add(std::make_shared<Relu>());
    m->add(std::make_shared<MaxPool2d>(P(3), P(2), P(1), P(1)));
    long long cin = 64, cout = 64;
    for (int i = 0; i < 4; ++i) {
        const long long stride = i == 0 ? 1 : 2;
        auto blk = std::make_shared<Sequential>();
        long long c = cin;
        for (int j = 0; j < 2; ++j) {
            blk->add(std::make_shared<BasicLayer>(c, cout, j == 0 ? stride : 1, batch_norm));
            c = cout;
        }
        m->add(blk);
        cin = cout;
        cout *= 2;
    }
    m->add(std::make_shared<AdaptiveAvgPool2d>(P(1)));
    m->add(std::make_shared<Flatten>());
    m->add(std::make_shared<Dense>(512, num_classes));
    return m;
}

// ---------------------------------------------------------------- DenseNet (models/densenet.rs)
struct BottleneckLayer : Layer {  // densenet.rs:121-157: relu, 1x1 conv to 4 x growth, 3x3 conv to growth; y joins x on the channel axis
    Sequential body;
    BottleneckLayer(long long in_planes, long long out_planes) {
        auto P = [](long long v) { return Pair{v, v}; };
        body.add(std::make_shared<Relu>());
        body.add(std::make_shared<Conv2d>(in_planes, out_planes * 4, P(1), P(1), P(0), P(1)));
        body.add(std::make_shared<Conv2d>(out_planes * 4, out_planes, P(3), P(1), P(1), P(1)));
    }
    Var pass(const Var &x) const override { return concat({x, body.pass(x)}, 3); }
    void params(std::vector<Var> *p) const override { body.params(p); }
};

std::shared_ptr<Sequential> densenet(long long chan_input, long long num_classes, long long depth, long long growth_rate) {
    auto P = [](long long v) { return Pair{v, v}; };
    if (depth < 10 || growth_rate < 1) shape_fail("densenet: depth must be at least 10 and the growth rate positive");
    long long in_planes = 2 * growth_rate;  // densenet.rs:58-84
    auto m = std::make_shared<Sequential>();
    m->add(std::make_shared<Conv2d>(chan_input, in_planes, P(3), P(1), P(1), P(1)));
    const long long n = (depth - 4) / 6;
    for (int i = 0; i < 3; ++i) {
        auto dense = std::make_shared<Sequential>();  // dense_layer, :96-106
        for (long long j = 0; j < n; ++j) dense->add(std::make_shared<BottleneckLayer>(in_planes + j * growth_rate, growth_rate));
        m->add(dense);
        in_planes += n * growth_rate;
        if (i < 2) {  // transition_layer, :86-94
            auto t = std::make_shared<Sequential>();
            t->add(std::make_shared<Relu>());
            t->add(std::make_shared<Conv2d>(in_planes, in_planes / 2, P(1), P(1), P(0), P(1)));
            t->add(std::make_shared<AvgPool2d>(P(2), P(2), P(0), P(1)));
            m->add(t);
            in_planes /= 2;
        }
    }
    m->add(std::make_shared<Relu>());
    m->add(std::make_shared<AdaptiveAvgPool2d>(P(1)));
    m->add(std::make_shared<Flatten>());
    m->add(std::make_shared<Dense>(in_planes, num_classes));
    return m;
}

// ---------------------------------------------------------------- MobileNetV2 (models/mobilenet.rs)
static long long make_divisible(long long val, long long div, long long min_val) {  // mobilenet.rs:10-18
    const long long v = std::max(min_val, (val + div / 2) / div * div);
    return (float)v < 0.9f * (float)val ? v + div : v;
}

struct InvertedResidual : Layer {  // mobilenet.rs:96-138
    Sequential body;
    bool residual;
    InvertedResidual(long long inp, long long oup, long long stride, long long expand_ratio) : residual(stride == 1 && inp == oup) {
        auto P = [](long long v) { return Pair{v, v}; };
        const long long hidden = inp * expand_ratio;
        if (expand_ratio != 1) {
            body.add(std::make_shared<Conv2d>(inp, hidden, P(1), P(1), P(0), P(1)));
            body.add(std::make_shared<Relu>());
        }
        // the reference passes padding 0 and dilation 0 here (mobilenet.rs:111): a full 3 x 3 convolution whose
        // nine taps all read the pixel at the window's corner
        body.add(std::make_shared<Conv2d>(hidden, hidden, P(3), P(stride), P(0), P(0)));
        body.add(std::make_shared<Relu>());
        body.add(std::make_shared<Conv2d>(hidden, oup, P(1), P(1), P(0), P(1)));
    }
    Var pass(const Var &x) const override { return residual ? add(x, body.pass(x)) : body.pass(x); }
    void params(std::vector<Var> *p) const override { body.params(p); }
};

std::shared_ptr<Sequential> mobilenet_v2(long long chan_in, long long num_classes) {  // mobilenet.rs:38-80, width_mul 1
    auto P = [](long long v) { return Pair{v, v}; };
    static const long long cfg[7][4] = {{1, 16, 1, 1}, {6, 24, 2, 2}, {6, 32, 3, 2}, {6, 64, 4, 2}, {6, 96, 3, 1}, {6, 160, 3, 2}, {6, 320, 1, 1}};
    long long c_in = make_divisible(32, 8, 8);
    auto m = std::make_shared<Sequential>();
    m->add(std::make_shared<Conv2d>(chan_in, c_in, P(3), P(2), P(1), P(1)));
    m->add(std::make_shared<Relu>());
    for (auto &row : cfg) {
        const long long c_out = make_divisible(row[1], 8, 8);
        for (long long i = 0; i < row[2]; ++i) {
            m->add(std::make_shared<InvertedResidual>(c_in, c_out, i == 0 ? row[3] : 1, row[0]));
            c_in = c_out;
        }
    }
    const long long last = make_divisible(1280, 8, 8);
    m->add(std::make_shared<Conv2d>(c_in, last, P(1), P(1), P(0), P(1)));  // Conv2d::new(in, out, 1): stride 1, padding 0, dilation 1
    m->add(std::make_shared<Relu>());
    m->add(std::make_shared<AdaptiveAvgPool2d>(P(1)));
    m->add(std::make_shared<Flatten>());
    m->add(std::make_shared<Dense>(last, num_classes));
    return m;
}

}  // namespace nn
}  // namespace sage
