"""numpy + C restatement of polygrad's CPU arithmetic for the execution path.

TEST INFRASTRUCTURE ONLY.  Only tests/, __graft_entry__.smoke() and the
cpu_baseline / reference legs of bench.py may import this module; the product
never does.  Parity: pinned -- tests/test_oracle.py checks every function here
against stock polygrad built from its own sources (oracle/_ref) where that
library is present, against the committed fixtures under tests/golden/ (made by
running stock polygrad; tests/golden/make_golden.py), and against polygrad's own
known-answer fixture test/fixtures/mlp_cross.json.

Each function states the polygrad construct it restates.  float32 throughout;
transcendental functions use libm where polygrad's CPU path uses polynomial
decompositions (src/codegen.c:2156-2679), which agree to a few ulp.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_port = None

F32 = np.float32
LOG2E = F32(1.0 / np.log(2.0))      # cf(1/M_LN2) rounded to float32, src/frontend.c:270-275


def port():
    """The C half (oracle/polyref_port.c), built by `make -C oracle port`."""
    global _port
    if _port is None:
        path = os.path.join(_HERE, 'libpolyref_port.so')
        if not os.path.isfile(path):
            raise FileNotFoundError(path + ' (run: make -C oracle port)')
        _port = ctypes.CDLL(path)
    return _port


def _fp(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


# ── elementwise (src/frontend.c:270-275, 479-493, 582-587, 603-613) ─────────
def exp(x):
    """poly_exp: exp2(x * (1/ln2))."""
    return np.exp2(x.astype(F32) * LOG2E).astype(F32)


def sigmoid(x):
    """poly_sigmoid: 1 / (1 + exp2(x * (-1/ln2)))."""
    x = x.astype(F32)
    with np.errstate(over='ignore'):
        e = np.exp2(x * (-LOG2E)).astype(F32)
    return (F32(1.0) / (F32(1.0) + e)).astype(F32)


def tanh(x):
    """poly_tanh_act: 2 * sigmoid(2x) - 1."""
    return (F32(2.0) * sigmoid(F32(2.0) * x.astype(F32)) - F32(1.0)).astype(F32)


def relu(x):
    """poly_relu: where(0 < x, x, 0)."""
    return np.where(F32(0) < x, x, F32(0)).astype(F32)


def gelu(x):
    """poly_gelu: 0.5 * x * (1 + tanh(sqrt(2/pi) * (x + 0.044715 * x^3)))."""
    x = x.astype(F32)
    x3 = x * (x * x)
    inner = x + F32(0.044715) * x3
    scaled = F32(np.sqrt(2.0 / np.pi)) * inner
    return (F32(0.5) * (x * (F32(1.0) + tanh(scaled)))).astype(F32)


# ── reductions over the last axis (src/frontend.c:921-992) ──────────────────
def _rows(x):
    x = np.ascontiguousarray(x, dtype=F32)
    return x.reshape(-1, x.shape[-1]), x.shape[:-1]


def row_sum(x):
    x2, lead = _rows(x)
    out = np.empty(x2.shape[0], F32)
    port().polyref_row_sum(_fp(x2), _fp(out), ctypes.c_int64(x2.shape[0]), ctypes.c_int64(x2.shape[1]))
    return out.reshape(lead)


def row_max(x):
    x2, lead = _rows(x)
    out = np.empty(x2.shape[0], F32)
    port().polyref_row_max(_fp(x2), _fp(out), ctypes.c_int64(x2.shape[0]), ctypes.c_int64(x2.shape[1]))
    return out.reshape(lead)


def row_mean(x):
    """poly_mean_reduce: sum / N in one kernel."""
    return (row_sum(x) / F32(x.shape[-1])).astype(F32)


def row_var(x, correction=1):
    """poly_var_reduce: two kernels, mean then sum((x-mean)^2) / (N - correction)."""
    x2, lead = _rows(x)
    mean = row_mean(x2)
    out = np.empty(x2.shape[0], F32)
    port().polyref_row_sqdev(_fp(x2), _fp(mean), _fp(out), ctypes.c_int64(x2.shape[0]), ctypes.c_int64(x2.shape[1]))
    return (out / F32(x.shape[-1] - correction)).astype(F32).reshape(lead)


def softmax(x):
    """poly_softmax (src/frontend.c:1131-1159): three kernels -- row max;
    sum of exp2((x-max)*log2e); exp2(...) / sum."""
    x = x.astype(F32)
    m = row_max(x)[..., None]
    e = exp(x - m)
    s = row_sum(e)[..., None]
    return (e / s).astype(F32)


def layernorm(x, eps=1e-5):
    """poly_layernorm (src/frontend.c:3585-3625): mean; biased variance;
    (x - mean) * (1 / sqrt(var + eps))."""
    x = x.astype(F32)
    mean = row_mean(x)[..., None]
    centered = x + (-mean)
    var = row_var(x, correction=0)[..., None]
    return (centered * (F32(1.0) / np.sqrt(var + F32(eps)))).astype(F32)


# ── contraction and gather ──────────────────────────────────────────────────
def matmul(a, b, bias=None, relu_out=False, bf16=False):
    """poly_dot (src/frontend.c:1029-1129) on 2-D operands: k ascending, unfused
    multiply and add in float32.  bf16=True rounds both operands to bfloat16 first."""
    a = np.asarray(a, dtype=F32)
    b = np.asarray(b, dtype=F32)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    out = np.empty((m, n), F32)
    fn = port().polyref_matmul_bf16 if bf16 else port().polyref_matmul_f32
    bp = _fp(np.ascontiguousarray(bias, dtype=F32)) if bias is not None else None
    I = ctypes.c_int64
    fn(_fp(a), _fp(b), _fp(out), I(m), I(n), I(k), I(a.strides[0] // 4), I(a.strides[1] // 4),
       I(b.strides[0] // 4), I(b.strides[1] // 4), bp, ctypes.c_int(int(relu_out)))
    return out


def embedding(ids, arange, table):
    """embedding() of src/modelzoo/models/gpt2.c:93-153: one-hot(ids == arange) . table."""
    ids = np.ascontiguousarray(ids, dtype=F32)
    arange = np.ascontiguousarray(arange, dtype=F32)
    table = np.ascontiguousarray(table, dtype=F32)
    v, d = table.shape
    out = np.empty((ids.size, d), F32)
    I = ctypes.c_int64
    port().polyref_embedding(_fp(ids.reshape(-1)), _fp(arange), _fp(table), _fp(out), I(ids.size), I(v), I(d))
    return out.reshape(ids.shape + (d,))


# ── models ──────────────────────────────────────────────────────────────────
def mlp_forward(x, weights, biases, activation='relu'):
    """poly_mlp_instance forward (src/model_mlp.c:203-245): x @ W.T + b with the
    activation between layers; weights are [out, in]."""
    h = np.asarray(x, dtype=F32)
    for i, (w, b) in enumerate(zip(weights, biases)):
        last = i == len(weights) - 1
        h = matmul(h, np.asarray(w, F32).T, bias=b, relu_out=(activation == 'relu' and not last))
    return h


def gpt2_forward(cfg, init, tokens, bf16=False):
    """poly_gpt2_build's forward graph (src/modelzoo/models/gpt2.c:320-526):
    one-hot embeddings, pre-LN blocks, full T x T attention with an additive
    -1e9 causal mask, tanh-GELU MLP, final LN, logits = h @ wte.T.
    `init(name, shape)` supplies parameters by polygrad's names."""
    V, D, H, L, T = cfg['vocab_size'], cfg['n_embd'], cfg['n_head'], cfg['n_layer'], cfg['max_seq_len']
    hd = D // H
    tokens = np.asarray(tokens, dtype=F32)
    B = tokens.shape[0]
    p = lambda name, *shape: init(name, shape)
    mm = lambda a, b, bias=None: matmul(a, b, bias=bias, bf16=bf16)
    wte, wpe = p('wte.weight', V, D), p('wpe.weight', T, D)
    tok = embedding(tokens, np.arange(V, dtype=F32), wte)                       # [B,T,D]
    pos = embedding(np.arange(T, dtype=F32)[None], np.arange(T, dtype=F32), wpe)  # [1,T,D]
    h = (tok + pos).astype(F32)
    ar = np.arange(T, dtype=F32)
    mask = np.where(ar[:, None] < ar[None, :], F32(-1e9), F32(0.0)).astype(F32)
    scale = F32(1.0 / np.sqrt(float(hd)))
    for i in range(L):
        pre = f'h.{i}.'
        ln1 = (layernorm(h) * p(pre + 'ln_1.weight', D) + p(pre + 'ln_1.bias', D)).astype(F32)
        qkv = mm(ln1.reshape(B * T, D), p(pre + 'attn.c_attn.weight', D, 3 * D),
                 p(pre + 'attn.c_attn.bias', 3 * D)).reshape(B, T, 3 * D)
        q, k, v = [qkv[..., j * D:(j + 1) * D].reshape(B, T, H, hd).transpose(0, 2, 1, 3) for j in range(3)]
        out = np.empty((B, H, T, hd), F32)
        for b in range(B):
            for hh in range(H):
                s = mm(q[b, hh], k[b, hh].T)
                s = (s * scale + mask).astype(F32)
                out[b, hh] = mm(softmax(s), v[b, hh])
        merged = out.transpose(0, 2, 1, 3).reshape(B * T, D)
        att = mm(merged, p(pre + 'attn.c_proj.weight', D, D), p(pre + 'attn.c_proj.bias', D)).reshape(B, T, D)
        h = (h + att).astype(F32)
        ln2 = (layernorm(h) * p(pre + 'ln_2.weight', D) + p(pre + 'ln_2.bias', D)).astype(F32)
        fc = mm(ln2.reshape(B * T, D), p(pre + 'mlp.c_fc.weight', D, 4 * D), p(pre + 'mlp.c_fc.bias', 4 * D))
        pr = mm(gelu(fc), p(pre + 'mlp.c_proj.weight', 4 * D, D), p(pre + 'mlp.c_proj.bias', D)).reshape(B, T, D)
        h = (h + pr).astype(F32)
    hf = (layernorm(h) * p('ln_f.weight', D) + p('ln_f.bias', D)).astype(F32)
    return mm(hf.reshape(B * T, D), wte.T).reshape(B, T, V)


def mlp_train_sgd(weights, biases, x, y, lr, steps, loss='mse'):
    """poly_instance_train_step with POLY_OPTIM_SGD on a ReLU MLP built by
    poly_mlp_instance: forward, the loss of src/model_mlp.c:269-304 as it
    evaluates (MSE: see the note in the code; cross-entropy: -mean over the batch of
    sum(target * log_softmax)), polygrad's autograd through it (src/autograd.c:
    relu passes the gradient where 0 < x) and p <- p - lr * grad
    (src/instance.c:1158-1162).  Returns the loss before each update and the
    final parameters.  float32 arithmetic; sums in numpy's order, which differs
    from the kernels' by rounding only."""
    ws = [np.array(w, dtype=F32) for w in weights]
    bs = [np.array(b, dtype=F32) for b in biases]
    x = np.asarray(x, dtype=F32)
    y = np.asarray(y, dtype=F32)
    lr = F32(lr)
    losses = []
    for _ in range(steps):
        acts, pre = [x], []
        for i, (w, b) in enumerate(zip(ws, bs)):
            z = (acts[-1] @ w.T + b).astype(F32)
            pre.append(z)
            acts.append(np.where(z > 0, z, F32(0)).astype(F32) if i + 1 < len(ws) else z)
        out = acts[-1]
        if loss == 'mse':
            # src/model_mlp.c:276-285 reduces axis 0 twice; a reduction keeps its axis (size 1), so
            # both run over the batch axis and the class axis is never summed.  The [1, out] result
            # is stored into the one-element loss buffer, which takes class 0: the loss polygrad
            # reports is sum_b (out[b, 0] - y[b, 0])^2 / (batch * out).  Autograd seeds every element
            # of that [1, out] value, so the gradient is the one of the full mean squared error.
            d = (out - y).astype(F32)
            losses.append(F32(np.sum(d[:, 0] * d[:, 0], dtype=F32) * F32(1.0 / d.size)))
            g = (d * F32(2.0) * F32(1.0 / d.size)).astype(F32)
        else:
            m = out.max(-1, keepdims=True)
            e = np.exp(out - m).astype(F32)
            s = e.sum(-1, keepdims=True, dtype=F32)
            logp = (out - m - np.log(s)).astype(F32)
            losses.append(F32(-np.sum(y * logp, dtype=F32) / F32(out.shape[0])))
            g = ((e / s) * y.sum(-1, keepdims=True) - y).astype(F32) / F32(out.shape[0])
        for i in range(len(ws) - 1, -1, -1):
            gw = (g.T @ acts[i]).astype(F32)
            gb = g.sum(0, dtype=F32)
            if i > 0:
                g = ((g @ ws[i]) * (pre[i - 1] > 0)).astype(F32)
            ws[i] = (ws[i] - lr * gw).astype(F32)
            bs[i] = (bs[i] - lr * gb).astype(F32)
    return np.array(losses, dtype=F32), ws, bs
