"""Seed-generated graphs with the shapes, sizes and value distributions of the benchmark
configurations.  They stand in for the real model files (ResNet-50, InSwapper-128, BERT-base),
which are not distributed with the reference either: its own model tests build synthetic
graphs the same way (tests/model_resnet.rs:66).

Every builder returns (graph, weights, feeds_fn) where feeds_fn(batch) gives the seeded input
tensors.  Graphs arrive in the form the reference's optimizer hands to an execution provider:
BatchNorm already folded into Conv with `activation="relu"` (fuse_conv_batchnorm /
fuse_conv_relu, root crate src/optimizer/fusion/conv/batchnorm.rs:17, relu.rs:69) and the
residual `Add -> Relu` left as two nodes.
"""
import numpy as np

from .graph import Graph, Node

SEED = 20261125


def _rng(tag):
    return np.random.default_rng([SEED] + [ord(c) for c in tag])


class _G:
    def __init__(self):
        self.nodes = []
        self.weights = {}

    def w(self, name, arr):
        self.weights[name] = np.ascontiguousarray(arr, dtype=np.float32)
        return name

    def node(self, op, inputs, outputs, name=None, **attrs):
        self.nodes.append(Node(op=op, name=name or f"{op}_{len(self.nodes)}", inputs=list(inputs), outputs=list(outputs), attrs=dict(attrs)))
        return outputs[0]


# ---------------------------------------------------------------------------------------------
# C1: INT8 MLP
# ---------------------------------------------------------------------------------------------
def build_int8_mlp(rows=64, dims=(1024, 4096, 4096, 1024), spelling="qlinearconv"):
    """QuantizeLinear (u8, scale 0.05, zp 128) -> 3 quantised linears -> DequantizeLinear.

    spelling "qlinearconv": each linear is a 1x1 QLinearConv on [rows, K, 1, 1], the only
    spelling inside the reference's operator set that carries per-output-channel weight
    scales and an int32 bias (its QLinearMatMul reads one b_scale lane and has no bias
    input: oxionnx-ops src/registry/quant_ops/qlinear_matmul.rs:230).
    spelling "qlinearmatmul": QLinearMatMul with a per-tensor weight scale and no bias.
    """
    g = _G()
    r = _rng("c1")
    g.w("x_scale", [0.05])
    g.w("x_zp", [128.0])
    cur = "x"
    if spelling == "qlinearconv":
        g.w("shape_in", [rows, dims[0], 1, 1])
        cur = g.node("Reshape", ["x", "shape_in"], ["x4"])
    cur = g.node("QuantizeLinear", [cur, "x_scale", "x_zp"], ["q0"])
    in_scale = "x_scale"
    for li in range(len(dims) - 1):
        k, n = dims[li], dims[li + 1]
        w_int = r.integers(-127, 128, size=(k, n)).astype(np.float32)
        w_scales = r.uniform(0.002, 0.02, size=n).astype(np.float32)
        bias = r.integers(-1000, 1001, size=n).astype(np.float32)
        g.w(f"y{li}_scale", [0.1])
        g.w(f"y{li}_zp", [128.0])
        if spelling == "qlinearconv":
            g.w(f"w{li}", w_int.T.reshape(n, k, 1, 1))
            g.w(f"w{li}_scale", w_scales)
            g.w(f"w{li}_zp", np.zeros(n))
            g.w(f"b{li}", bias)
            cur = g.node("QLinearConv", [cur, in_scale, "x_zp" if li == 0 else f"y{li-1}_zp", f"w{li}", f"w{li}_scale", f"w{li}_zp",
                                          f"y{li}_scale", f"y{li}_zp", f"b{li}"], [f"q{li+1}"], name=f"linear{li}")
        else:
            g.w(f"w{li}", w_int)
            g.w(f"w{li}_scale", [float(w_scales.mean())])
            g.w(f"w{li}_zp", [0.0])
            cur = g.node("QLinearMatMul", [cur, in_scale, "x_zp" if li == 0 else f"y{li-1}_zp", f"w{li}", f"w{li}_scale", f"w{li}_zp",
                                            f"y{li}_scale", f"y{li}_zp"], [f"q{li+1}"], name=f"linear{li}")
        in_scale = f"y{li}_scale"
    last = len(dims) - 2
    cur = g.node("DequantizeLinear", [cur, f"y{last}_scale", f"y{last}_zp"], ["y4" if spelling == "qlinearconv" else "y"])
    if spelling == "qlinearconv":
        g.w("shape_out", [rows, dims[-1]])
        cur = g.node("Reshape", [cur, "shape_out"], ["y"])
    graph = Graph(nodes=g.nodes, input_names=["x"], output_names=["y"])

    def feeds(batch=rows, seed_tag="c1_in"):
        return {"x": _rng(seed_tag).standard_normal((rows, dims[0])).astype(np.float32)}

    macs = rows * sum(dims[i] * dims[i + 1] for i in range(len(dims) - 1))
    return graph, g.weights, feeds, dict(ops=2.0 * macs, rows=rows)


# ---------------------------------------------------------------------------------------------
# ResNet-50 v1.5 topology (float: C2, QLinearConv: C5)
# ---------------------------------------------------------------------------------------------
def _resnet_plan(base=64, blocks=(3, 4, 6, 3)):
    """[(in, mid, out, stride)] per bottleneck, stride on the 3x3 (v1.5)."""
    plan = []
    cin = base
    for si, nb in enumerate(blocks):
        mid = base * (2 ** si)
        out = mid * 4
        for bi in range(nb):
            plan.append((cin, mid, out, 2 if (bi == 0 and si > 0) else 1, bi == 0))
            cin = out
    return plan


def _conv_out(size, k, s, p):
    return (size + 2 * p - k) // s + 1


def fold_batchnorm(w, b, gamma, beta, mean, var, eps):
    """fuse_conv_batchnorm's arithmetic (src/optimizer/fusion/conv/batchnorm.rs:126-144), in f32 like the reference:
    inv_std = 1 / sqrt(var + eps); factor = gamma * inv_std; W' = W * factor per output channel; b' = (b - mean) * factor + beta, with b = 0
    when the convolution has no bias."""
    f32 = np.float32
    factor = (gamma.astype(f32) * (f32(1.0) / np.sqrt(var.astype(f32) + f32(eps)))).astype(f32)
    b = np.zeros(w.shape[0], f32) if b is None else b.astype(f32)
    return (w.astype(f32) * factor.reshape((-1,) + (1,) * (w.ndim - 1))).astype(f32), ((b - mean.astype(f32)) * factor + beta.astype(f32)).astype(f32)


def build_resnet50_f32(batch=32, image=224, base=64, blocks=(3, 4, 6, 3), classes=1000):
    """ResNet-50 v1.5, BatchNorm folded into the convolutions, fused ReLU."""
    g = _G()
    r = _rng("c2")
    macs = [0]

    def conv(x, cin, cout, ksz, stride, pad, relu, hw, name):
        fan_in = cin * ksz * ksz
        w = r.standard_normal((cout, cin, ksz, ksz)).astype(np.float32) * np.float32(np.sqrt(2.0 / fan_in))
        gamma = r.uniform(0.5, 1.5, cout).astype(np.float32)
        beta = (r.standard_normal(cout) * 0.1).astype(np.float32)
        mean = (r.standard_normal(cout) * 0.1).astype(np.float32)
        var = r.uniform(0.5, 1.5, cout).astype(np.float32)
        fw, fb = fold_batchnorm(w, None, gamma, beta, mean, var, 1e-5)
        g.w(f"{name}_out_fused_weight", fw)
        g.w(f"{name}_out_fused_bias", fb)
        attrs = dict(strides=[stride, stride], pads=[pad, pad, pad, pad], dilations=[1, 1], group=1, kernel_shape=[ksz, ksz])
        if relu:
            attrs["activation"] = "relu"
        out_hw = _conv_out(hw, ksz, stride, pad)
        macs[0] += out_hw * out_hw * cout * fan_in
        return g.node("Conv", [x, f"{name}_out_fused_weight", f"{name}_out_fused_bias"], [f"{name}_out"], name=f"{name}_fused_convbn", **attrs), out_hw

    hw = image
    x, hw = conv("input", 3, base, 7, 2, 3, True, hw, "stem")
    x = g.node("MaxPool", [x], ["pool_out"], name="pool", kernel_shape=[3, 3], strides=[2, 2], pads=[1, 1, 1, 1])
    hw = _conv_out(hw, 3, 2, 1)
    for bi, (cin, mid, cout, stride, first) in enumerate(_resnet_plan(base, blocks)):
        name = f"b{bi}"
        identity = x
        y, _ = conv(x, cin, mid, 1, 1, 0, True, hw, f"{name}_c1")
        y, hw2 = conv(y, mid, mid, 3, stride, 1, True, hw, f"{name}_c2")
        y, _ = conv(y, mid, cout, 1, 1, 0, False, hw2, f"{name}_c3")
        if first:
            identity, _ = conv(x, cin, cout, 1, stride, 0, False, hw, f"{name}_sc")
        s = g.node("Add", [y, identity], [f"{name}_sum"], name=f"{name}_add")
        x = g.node("Relu", [s], [f"{name}_relu"], name=f"{name}_act")
        hw = hw2
    feat = base * (2 ** (len(blocks) - 1)) * 4
    x = g.node("GlobalAveragePool", [x], ["gap"], name="gap")
    x = g.node("Flatten", [x], ["flat"], name="flatten", axis=1)
    g.w("fc_weight", r.standard_normal((classes, feat)).astype(np.float32) * np.float32(np.sqrt(1.0 / feat)))
    g.w("fc_bias", (r.standard_normal(classes) * 0.01).astype(np.float32))
    macs[0] += feat * classes
    g.node("Gemm", [x, "fc_weight", "fc_bias"], ["logits"], name="fc", alpha=1.0, beta=1.0, transB=1)
    graph = Graph(nodes=g.nodes, input_names=["input"], output_names=["logits"])

    def feeds(b=batch, seed_tag="c2_in"):
        return {"input": _rng(seed_tag).standard_normal((b, 3, image, image)).astype(np.float32)}

    return graph, g.weights, feeds, dict(ops=2.0 * macs[0] * batch, macs_per_image=macs[0], batch=batch)


def build_resnet50_qlinear(batch=128, image=224, base=64, blocks=(3, 4, 6, 3), classes=1000, typed_input=False):
    """The same topology as QLinearConv nodes: u8 activations (first scale fitted to N(0,1),
    zero point 128), i8 per-output-channel weights U[-127,127] with scales U[0.001,0.01], int32
    biases, output zero point 0 behind a ReLU (spelled as an explicit Relu node on the quantised
    lanes, so the reference's value-based saturation inference and the ONNX typed semantics
    agree), residual joins as DequantizeLinear -> Add -> Relu -> QuantizeLinear.

    typed_input: the graph input is the already quantised image, declared and fed as u8 lanes
    (`input_q`, a quarter of the bytes of the f32 image); the QuantizeLinear of the f32 form is
    then done by the feed generator with the same arithmetic, so both forms see the same lanes."""
    g = _G()
    r = _rng("c5")
    macs = [0]
    g.w("zp0", [0.0])
    g.w("zp128", [128.0])

    def qconv(x, x_scale, x_zp_name, x_std, cin, cout, ksz, stride, pad, relu, hw, name):
        k = cin * ksz * ksz
        w = r.integers(-127, 128, size=(cout, cin, ksz, ksz)).astype(np.float32)
        ws = r.uniform(0.001, 0.01, cout).astype(np.float32)
        bias = r.integers(-1000, 1001, size=cout).astype(np.float32)
        # analytic spread of the real-valued output, used only to pick a non-degenerate y_scale
        out_std = float(x_std * 73.3 * float(ws.mean()) * np.sqrt(k))
        y_scale = np.float32(out_std * (3.0 / 255.0 if relu else 6.0 / 255.0))
        g.w(f"{name}_w", w)
        g.w(f"{name}_ws", ws)
        g.w(f"{name}_wzp", np.zeros(cout))
        g.w(f"{name}_b", bias)
        g.w(f"{name}_ys", [y_scale])
        out_hw = _conv_out(hw, ksz, stride, pad)
        macs[0] += out_hw * out_hw * cout * k
        y = g.node("QLinearConv", [x, x_scale, x_zp_name, f"{name}_w", f"{name}_ws", f"{name}_wzp", f"{name}_ys", "zp0" if relu else "zp128",
                                   f"{name}_b"], [f"{name}_q"], name=name, strides=[stride, stride], pads=[pad, pad, pad, pad], dilations=[1, 1],
                   group=1, kernel_shape=[ksz, ksz])
        if relu:
            y = g.node("Relu", [y], [f"{name}_qr"], name=f"{name}_relu")
        return y, f"{name}_ys", out_hw, (out_std * 0.6 if relu else out_std)

    g.w("in_scale", [np.float32(4.0 / 127.0)])
    if typed_input:
        x = "input_q"
    else:
        x = g.node("QuantizeLinear", ["input", "in_scale", "zp128"], ["input_q"], name="quantize_input")
    hw = image
    x, xs, hw, std = qconv(x, "in_scale", "zp128", 1.0, 3, base, 7, 2, 3, True, hw, "stem")
    x = g.node("MaxPool", [x], ["pool_q"], name="pool", kernel_shape=[3, 3], strides=[2, 2], pads=[1, 1, 1, 1])
    hw = _conv_out(hw, 3, 2, 1)
    xzp = "zp0"
    for bi, (cin, mid, cout, stride, first) in enumerate(_resnet_plan(base, blocks)):
        name = f"b{bi}"
        y, ys1, _, s1 = qconv(x, xs, xzp, std, cin, mid, 1, 1, 0, True, hw, f"{name}_c1")
        y, ys2, hw2, s2 = qconv(y, ys1, "zp0", s1, mid, mid, 3, stride, 1, True, hw, f"{name}_c2")
        y, ys3, _, s3 = qconv(y, ys2, "zp0", s2, mid, cout, 1, 1, 0, False, hw2, f"{name}_c3")
        if first:
            sc, scs, _, ssc = qconv(x, xs, xzp, std, cin, cout, 1, stride, 0, False, hw, f"{name}_sc")
            sc_zp = "zp128"
        else:
            sc, scs, ssc, sc_zp = x, xs, std, xzp
        a = g.node("DequantizeLinear", [y, ys3, "zp128"], [f"{name}_dq_main"], name=f"{name}_dq_main")
        b = g.node("DequantizeLinear", [sc, scs, sc_zp], [f"{name}_dq_short"], name=f"{name}_dq_short")
        s = g.node("Add", [a, b], [f"{name}_sum"], name=f"{name}_add")
        s = g.node("Relu", [s], [f"{name}_relu"], name=f"{name}_act")
        join_std = float(np.sqrt(s3 * s3 + ssc * ssc)) * 0.6
        g.w(f"{name}_js", [np.float32(join_std * 4.0 / 127.0)])
        x = g.node("QuantizeLinear", [s, f"{name}_js", "zp0"], [f"{name}_out_q"], name=f"{name}_requant")
        # The weight scales of this configuration (U[0.001, 0.01] on U[-127,127] weights) are not
        # variance-preserving, so a consistently labelled real domain grows by a few x per layer and
        # would leave the f32 range over 50 layers.  Each block output is therefore re-labelled with
        # a fixed scale for its consumers; the integer lanes, which are what is compared, keep a
        # healthy spread either way.
        g.w(f"{name}_xs", [np.float32(0.02)])
        xs, xzp, std, hw = f"{name}_xs", "zp0", 0.02 * 32.0, hw2
    feat = base * (2 ** (len(blocks) - 1)) * 4
    d = g.node("DequantizeLinear", [x, xs, "zp0"], ["tail_dq"], name="tail_dq")
    p = g.node("GlobalAveragePool", [d], ["gap"], name="gap")
    g.w("gap_scale", [np.float32(std * 4.0 / 127.0 / 2.0)])
    q = g.node("QuantizeLinear", [p, "gap_scale", "zp128"], ["gap_q"], name="gap_quant")
    fc, fcs, _, _ = qconv(q, "gap_scale", "zp128", std / 2.0, feat, classes, 1, 1, 0, False, 1, "fc")
    o = g.node("DequantizeLinear", [fc, fcs, "zp128"], ["fc_dq"], name="fc_dq")
    g.node("Flatten", [o], ["logits"], name="flatten", axis=1)
    graph = Graph(nodes=g.nodes, input_names=["input_q" if typed_input else "input"], output_names=["logits"])

    def feeds(b=batch, seed_tag="c5_in"):
        x = _rng(seed_tag).standard_normal((b, 3, image, image)).astype(np.float32)
        if not typed_input:
            return {"input": x}
        # QuantizeLinear(scale 4/127, zero point 128) in f32: divide, round half to even, add, saturate
        q = np.rint(x / np.float32(4.0 / 127.0)).astype(np.float32) + np.float32(128.0)
        return {"input_q": np.clip(q, 0.0, 255.0).astype(np.uint8)}

    return graph, g.weights, feeds, dict(ops=2.0 * macs[0] * batch, macs_per_image=macs[0], batch=batch)


# ---------------------------------------------------------------------------------------------
# C3: InSwapper-128-shaped face-swap generator (float)
# ---------------------------------------------------------------------------------------------
def build_inswapper_f32(batch=16, size=128, widths=(128, 256, 512, 1024), blocks=6, latent=512):
    """Encoder, `blocks` residual style blocks, decoder, 7x7 + Tanh, in the form the reference's
    optimizer hands to an execution provider: the layer inventory of its own InSwapper parity
    test (oxionnx-gpu/tests/c3_conv2d_parity.rs:80-164: 7x7 3->128 on the reflect-padded 134^2
    image, 3x3 128->256, 3x3 stride 2 to 512 and to 1024, twelve pad-free 3x3 1024->1024 on
    reflect-padded 34^2 maps, 3x3 1024->512 at 64^2, 512->256 and 256->128 at 128^2, 7x7 128->3),
    every instance normalisation already fused into `OxiInstanceNorm` (epsilon 1e-8,
    src/optimizer/fusion/instance_norm.rs:17,199) and followed by separate per-sample
    Mul(scale[N,C,1,1]) and Add(shift[N,C,1,1]) nodes (instance_norm.rs:23-26) whose operands
    come from one Gemm(latent -> 2*C) per normalisation.  Inputs: target image ~U[0,1], latent
    ~N(0,1) L2-normalised per row.  Random-initialised weights stand in for the real model."""
    g = _G()
    r = _rng("c3")
    macs = [0]
    w0, w1, w2, w3 = widths

    def conv(x, cin, cout, ksz, stride, pad, relu, hw, name):
        fan_in = cin * ksz * ksz
        g.w(f"{name}_w", r.standard_normal((cout, cin, ksz, ksz)).astype(np.float32) * np.float32(np.sqrt(2.0 / fan_in)))
        g.w(f"{name}_b", (r.standard_normal(cout) * 0.05).astype(np.float32))
        attrs = dict(strides=[stride, stride], pads=[pad] * 4, dilations=[1, 1], group=1, kernel_shape=[ksz, ksz])
        if relu:
            attrs["activation"] = "relu"
        out_hw = _conv_out(hw, ksz, stride, pad)
        macs[0] += out_hw * out_hw * cout * fan_in
        return g.node("Conv", [x, f"{name}_w", f"{name}_b"], [f"{name}_out"], name=name, **attrs), out_hw

    def reflect(x, p, name):
        g.w(f"{name}_pads", [0, 0, p, p, 0, 0, p, p])
        return g.node("Pad", [x, f"{name}_pads"], [f"{name}_out"], name=name, mode="reflect")

    def adain(x, c, name):
        """OxiInstanceNorm -> Mul(scale) -> Add(shift), scale/shift from one Gemm on the latent."""
        g.w(f"{name}_fc_w", r.standard_normal((2 * c, latent)).astype(np.float32) * np.float32(np.sqrt(1.0 / latent)))
        fc_b = np.concatenate([np.ones(c, np.float32), np.zeros(c, np.float32)]) + (r.standard_normal(2 * c) * 0.02).astype(np.float32)
        g.w(f"{name}_fc_b", fc_b)
        macs[0] += 2 * c * latent
        style = g.node("Gemm", ["latent", f"{name}_fc_w", f"{name}_fc_b"], [f"{name}_style"], name=f"{name}_fc", alpha=1.0, beta=1.0, transB=1)
        g.w(f"{name}_s0", [0]), g.w(f"{name}_s1", [c]), g.w(f"{name}_e1", [2 * c]), g.w(f"{name}_ax", [1]), g.w(f"{name}_shape", [-1, c, 1, 1])
        sc = g.node("Slice", [style, f"{name}_s0", f"{name}_s1", f"{name}_ax"], [f"{name}_scale2d"], name=f"{name}_slice_scale")
        sh = g.node("Slice", [style, f"{name}_s1", f"{name}_e1", f"{name}_ax"], [f"{name}_shift2d"], name=f"{name}_slice_shift")
        sc = g.node("Reshape", [sc, f"{name}_shape"], [f"{name}_scale"], name=f"{name}_reshape_scale")
        sh = g.node("Reshape", [sh, f"{name}_shape"], [f"{name}_shift"], name=f"{name}_reshape_shift")
        y = g.node("OxiInstanceNorm", [x], [f"{name}_norm"], name=f"{name}_in", epsilon=1e-8)
        y = g.node("Mul", [y, sc], [f"{name}_mul"], name=f"{name}_mul")
        return g.node("Add", [y, sh], [f"{name}_mod"], name=f"{name}_add")

    hw = size
    x = reflect("target", 3, "enc0_pad")
    x, hw = conv(x, 3, w0, 7, 1, 0, True, hw + 6, "enc0")
    x, hw = conv(x, w0, w1, 3, 1, 1, True, hw, "enc1")
    x, hw = conv(x, w1, w2, 3, 2, 1, True, hw, "enc2")
    x, hw = conv(x, w2, w3, 3, 2, 1, True, hw, "enc3")
    for bi in range(blocks):
        name = f"s{bi}"
        y = reflect(x, 1, f"{name}_pad1")
        y, _ = conv(y, w3, w3, 3, 1, 0, False, hw + 2, f"{name}_c1")
        y = adain(y, w3, f"{name}_a1")
        y = g.node("Relu", [y], [f"{name}_relu"], name=f"{name}_act")
        y = reflect(y, 1, f"{name}_pad2")
        y, _ = conv(y, w3, w3, 3, 1, 0, False, hw + 2, f"{name}_c2")
        y = adain(y, w3, f"{name}_a2")
        x = g.node("Add", [y, x], [f"{name}_sum"], name=f"{name}_res")
    g.w("up_scales", [1, 1, 2, 2])
    up = dict(mode="linear", coordinate_transformation_mode="half_pixel")
    x = g.node("Resize", [x, "", "up_scales"], ["up1"], name="up1", **up)
    hw *= 2
    x, hw = conv(x, w3, w2, 3, 1, 1, True, hw, "dec1")
    x = g.node("Resize", [x, "", "up_scales"], ["up2"], name="up2", **up)
    hw *= 2
    x, hw = conv(x, w2, w1, 3, 1, 1, True, hw, "dec2")
    x, hw = conv(x, w1, w0, 3, 1, 1, True, hw, "dec3")
    x = reflect(x, 3, "out_pad")
    x, hw = conv(x, w0, 3, 7, 1, 0, False, hw + 6, "out_conv")
    g.node("Tanh", [x], ["image"], name="out_tanh")
    graph = Graph(nodes=g.nodes, input_names=["target", "latent"], output_names=["image"])

    def feeds(b=batch, seed_tag="c3_in"):
        rr = _rng(seed_tag)
        target = rr.uniform(0.0, 1.0, (b, 3, size, size)).astype(np.float32)
        z = rr.standard_normal((b, latent)).astype(np.float32)
        z /= np.sqrt(np.sum(z.astype(np.float64) ** 2, axis=1, keepdims=True)).astype(np.float32)
        return {"target": target, "latent": z}

    return graph, g.weights, feeds, dict(ops=2.0 * macs[0] * batch, macs_per_image=macs[0], batch=batch)


# ---------------------------------------------------------------------------------------------
# C4: BERT-base-shaped encoder, dynamic INT8 linears
# ---------------------------------------------------------------------------------------------
def build_bert_dynamic_int8(batch=64, seq=128, hidden=768, heads=12, ffn=3072, layers=12, vocab=30522):
    """Token ids uniform in [0, vocab), attention mask all ones.  Every linear is
    DynamicQuantizeLinear (u8, per tensor: quant_ops/dynamic_quantize.rs:40-94) -> MatMulInteger
    (i8 per-output-channel weights ~ round(N(0, 40)) clipped to +-127, zero point 0;
    qlinear_matmul.rs:181-199) -> Cast -> Mul(x_scale * w_scale[n]) -> Add(bias), the chain a
    dynamically quantised export spells; LayerNormalization, Softmax, Gelu and the two attention
    products stay in f32.  Returns the last hidden state [batch, seq, hidden]."""
    g = _G()
    r = _rng("c4")
    macs = [0]
    d_head = hidden // heads
    g.w("word_emb", (r.standard_normal((vocab, hidden)) * 0.05).astype(np.float32))
    g.w("pos_emb", (r.standard_normal((seq, hidden)) * 0.05).astype(np.float32))
    g.w("type_emb", (r.standard_normal(hidden) * 0.05).astype(np.float32))
    g.w("one", [1.0]), g.w("mask_scale", [-10000.0]), g.w("mask_shape", [batch, 1, 1, seq]), g.w("att_scale", [1.0 / np.sqrt(d_head)])
    g.w("rows_shape", [batch * seq, hidden]), g.w("heads_shape", [batch, seq, heads, d_head]), g.w("out_shape", [batch, seq, hidden])

    def layer_norm(x, name):
        g.w(f"{name}_g", r.uniform(0.8, 1.2, hidden).astype(np.float32))
        g.w(f"{name}_b", (r.standard_normal(hidden) * 0.05).astype(np.float32))
        return g.node("LayerNormalization", [x, f"{name}_g", f"{name}_b"], [f"{name}_out"], name=name, axis=-1, epsilon=1e-12)

    def quantise(x, name):
        g.node("DynamicQuantizeLinear", [x], [f"{name}_q", f"{name}_s", f"{name}_z"], name=name)
        return f"{name}_q", f"{name}_s", f"{name}_z"

    def linear(xq, xs, xz, k, n, name):
        wq = np.clip(np.rint(r.standard_normal((k, n)) * 40.0), -127, 127).astype(np.float32)
        g.w(f"{name}_w", wq)
        g.w(f"{name}_ws", r.uniform(0.0005, 0.002, n).astype(np.float32) * np.float32(np.sqrt(768.0 / k)))
        g.w(f"{name}_bias", (r.standard_normal(n) * 0.02).astype(np.float32))
        macs[0] += seq * k * n
        acc = g.node("MatMulInteger", [xq, f"{name}_w", xz], [f"{name}_acc"], name=f"{name}_mmi")
        accf = g.node("Cast", [acc], [f"{name}_accf"], name=f"{name}_cast", to=1)
        sc = g.node("Mul", [xs, f"{name}_ws"], [f"{name}_scale"], name=f"{name}_scales")
        y = g.node("Mul", [accf, sc], [f"{name}_scaled"], name=f"{name}_rescale")
        return g.node("Add", [y, f"{name}_bias"], [f"{name}_out"], name=f"{name}_addb")

    emb = g.node("Gather", ["word_emb", "input_ids"], ["emb_word"], name="emb_gather", axis=0)
    emb = g.node("Add", [emb, "pos_emb"], ["emb_pos"], name="emb_add_pos")
    emb = g.node("Add", [emb, "type_emb"], ["emb_sum"], name="emb_add_type")
    x = layer_norm(emb, "emb_ln")
    x = g.node("Reshape", [x, "rows_shape"], ["x0"], name="rows")
    m = g.node("Sub", ["one", "attention_mask"], ["mask_inv"], name="mask_inv")
    m = g.node("Mul", [m, "mask_scale"], ["mask_add"], name="mask_scale_mul")
    mask = g.node("Reshape", [m, "mask_shape"], ["mask4"], name="mask_reshape")
    for li in range(layers):
        p = f"l{li}"
        xq, xs, xz = quantise(x, f"{p}_qx")
        q = linear(xq, xs, xz, hidden, hidden, f"{p}_q")
        k = linear(xq, xs, xz, hidden, hidden, f"{p}_k")
        v = linear(xq, xs, xz, hidden, hidden, f"{p}_v")
        q4 = g.node("Transpose", [g.node("Reshape", [q, "heads_shape"], [f"{p}_q4r"], name=f"{p}_q_split")], [f"{p}_q4"], name=f"{p}_q_t", perm=[0, 2, 1, 3])
        k4 = g.node("Transpose", [g.node("Reshape", [k, "heads_shape"], [f"{p}_k4r"], name=f"{p}_k_split")], [f"{p}_k4t"], name=f"{p}_k_t", perm=[0, 2, 3, 1])
        v4 = g.node("Transpose", [g.node("Reshape", [v, "heads_shape"], [f"{p}_v4r"], name=f"{p}_v_split")], [f"{p}_v4"], name=f"{p}_v_t", perm=[0, 2, 1, 3])
        s = g.node("MatMul", [q4, k4], [f"{p}_scores"], name=f"{p}_qk")
        s = g.node("Mul", [s, "att_scale"], [f"{p}_scores_scaled"], name=f"{p}_scale")
        s = g.node("Add", [s, mask], [f"{p}_scores_masked"], name=f"{p}_mask")
        pr = g.node("Softmax", [s], [f"{p}_probs"], name=f"{p}_softmax", axis=-1)
        c = g.node("MatMul", [pr, v4], [f"{p}_ctx4"], name=f"{p}_av")
        macs[0] += 2 * heads * seq * seq * d_head
        c = g.node("Transpose", [c], [f"{p}_ctx_t"], name=f"{p}_ctx_merge_t", perm=[0, 2, 1, 3])
        c = g.node("Reshape", [c, "rows_shape"], [f"{p}_ctx"], name=f"{p}_ctx_merge")
        cq, cs, cz = quantise(c, f"{p}_qc")
        o = linear(cq, cs, cz, hidden, hidden, f"{p}_o")
        x1 = layer_norm(g.node("Add", [o, x], [f"{p}_res1"], name=f"{p}_add1"), f"{p}_ln1")
        hq, hs, hz = quantise(x1, f"{p}_qh")
        h = linear(hq, hs, hz, hidden, ffn, f"{p}_f1")
        h = g.node("Gelu", [h], [f"{p}_gelu"], name=f"{p}_act")
        fq, fs, fz = quantise(h, f"{p}_qf")
        f2 = linear(fq, fs, fz, ffn, hidden, f"{p}_f2")
        x = layer_norm(g.node("Add", [f2, x1], [f"{p}_res2"], name=f"{p}_add2"), f"{p}_ln2")
    g.node("Reshape", [x, "out_shape"], ["hidden"], name="out_reshape")
    graph = Graph(nodes=g.nodes, input_names=["input_ids", "attention_mask"], output_names=["hidden"])

    def feeds(b=batch, seed_tag="c4_in"):
        rr = _rng(seed_tag)
        return {"input_ids": rr.integers(0, vocab, (b, seq)).astype(np.float32), "attention_mask": np.ones((b, seq), np.float32)}

    return graph, g.weights, feeds, dict(ops=2.0 * macs[0] * batch, macs_per_sequence=macs[0], batch=batch, tokens=batch * seq)
