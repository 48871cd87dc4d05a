"""Plain, slow restatement of the Dugalix decoder (torch on the CPU, float32 or float64), one function per mechanism.

It shares no code with the CUDA path: the tests build small random checkpoints, run both and compare. A sequence is processed
whole, token loops where the design is recurrent, no cache and no state object.

Notation: x residual stream [T, W]; N(v; g) = v / sqrt(mean(v^2) + eps) * (1 + g). A layer is
    u = shift(N(x; g1));  x <- x + r * N(mixer(u); g1b);  x <- x + r * N(ff(N(x; g2)); g2b)
with r = residual_mult and shift(h)_t = h_t + (h_(t-1) - h_t) * s (h_(-1) = 0, s one number per channel). Mixers:
  'attention'  grouped-query attention whose values are the un-rotated keys, a sliding window, and sigmoid(score + b_head)
               as the weight of a visible key (no normalisation over keys);
  'parallel'   a_l * softmax attention (window that also keeps the first tokens, biases, linearly slowed rotation)
               + a_r * matrix-memory recurrence (exponential input gate, sigmoid forget gate, running-maximum stabiliser).
Feed-forwards: dense relu^2 unit, or a mixture: softmax router over real and identity experts, choice by corrected scores inside
the best groups, un-renormalised weights, plus an always-on shared unit behind a per-token sigmoid gate.
cfg is the parsed config.json (a dict), w the tensor dict of the checkpoint.
"""
import math
import torch


def norm1p(v, g, eps):
    """v / rms(v) * (1 + g): the gain is stored around zero"""
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * (1.0 + g)


def unit_rms(v, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def token_shift(h, s):
    """h_t + (h_(t-1) - h_t) * s with zeros before the first token"""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return h + (prev - h) * s


def relu2(z):
    return torch.relu(z) ** 2


def rot_frequencies(rot, dtype=torch.float64):
    """pair i of the rotated dims turns by base^(-2i/dims) per position, divided by scaling.factor when there is one"""
    dims = int(rot['dims'])
    f = float(rot['base']) ** (-2.0 * torch.arange(dims // 2, dtype=dtype) / dims)
    sc = rot.get('scaling')
    if sc:
        f = f / float(sc['factor'])
    return f


def rotate(v, pos, rot):
    """v [T, heads, d]: dims i and i + dims/2 (i < dims/2) of the leading `dims` numbers turn by pos * f_i, the rest stays"""
    if not rot:
        return v
    dims = int(rot['dims'])
    half = dims // 2
    ang = pos.to(v.dtype)[:, None] * rot_frequencies(rot, v.dtype)[None, :]          # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], -1)


def visible(T, size, keep_first=0):
    """[T, T] bool: query i sees key j when j <= i and (i - j < size or j < keep_first); size 0 = no window"""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    near = (i - j < size) if size else torch.ones(T, T, dtype=torch.bool)
    return (j <= i) & (near | (j < keep_first))


def softmax_window_attention(u, w, p, mc):
    """the left half of a 'parallel' mixer: biased projections, rotation, window with kept first tokens, softmax"""
    T = u.shape[0]
    H, G, d, dv = int(mc['heads']), int(mc.get('kv_heads', mc['heads'])), int(mc['dim']), int(mc.get('vdim', mc['dim']))
    lin = lambda n: u @ w[p + n].to(u.dtype).T + w[p + n + '.b'].to(u.dtype)
    pos = torch.arange(T)
    q = rotate(lin('q').view(T, H, d), pos, mc.get('rot'))
    k = rotate(lin('k').view(T, G, d), pos, mc.get('rot'))
    v = lin('v').view(T, G, dv)
    mask = mc.get('mask') or {}
    vis = visible(T, int(mask.get('size', 0) or 0), int(mask.get('keep_first', 0) or 0))
    out = torch.zeros(T, H, dv, dtype=u.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * float(mc['scale'])
        s = s.masked_fill(~vis, float('-inf'))
        out[:, h] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * dv) @ w[p + 'o'].to(u.dtype).T + w[p + 'o.b'].to(u.dtype)


def sigmoid_window_attention(u, w, p, mc):
    """'attention' mixer: values are the keys before rotation; weight of a visible key = sigmoid(score + b_head)"""
    T = u.shape[0]
    H, G, d = int(mc['heads']), int(mc.get('kv_heads', mc['heads'])), int(mc['dim'])
    pos = torch.arange(T)
    q = rotate((u @ w[p + 'q'].to(u.dtype).T).view(T, H, d), pos, mc.get('rot'))
    k_plain = (u @ w[p + 'k'].to(u.dtype).T).view(T, G, d)
    k = rotate(k_plain, pos, mc.get('rot'))
    vis = visible(T, int((mc.get('mask') or {}).get('size', 0) or 0))
    pb = w[p + 'pb'].to(u.dtype)
    out = torch.zeros(T, H, d, dtype=u.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * float(mc['scale']) + pb[h]
        out[:, h] = (torch.sigmoid(s) * vis) @ k_plain[:, g]
    return out.reshape(T, H * d) @ w[p + 'o'].to(u.dtype).T


def matrix_memory(u, w, p, mc, eps):
    """the right half of a 'parallel' mixer, token by token. Per head: memory S [d, dv], normaliser n [d], stabiliser m (starts
    at 0). log gates: a_t = cap tanh(pre_i / cap), b_t = logsigmoid(cap tanh(pre_f / cap));
    m_t = max(b_t + m_(t-1), a_t); S_t = e^(b_t + m_(t-1) - m_t) S_(t-1) + e^(a_t - m_t) k_t v_t^T, n_t alike with k_t;
    y_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)."""
    T = u.shape[0]
    H, d, dv, cap = int(mc['heads']), int(mc['dim']), int(mc.get('vdim', mc['dim'])), float(mc['gate_cap'])
    lin = lambda n: u @ w[p + n].to(u.dtype).T
    q = lin('q').view(T, H, d) * d ** -0.5
    k = lin('k').view(T, H, d)
    v = lin('v').view(T, H, dv)
    a = cap * torch.tanh((lin('i') + w[p + 'i.b'].to(u.dtype)) / cap)                              # [T, H]
    b = torch.nn.functional.logsigmoid(cap * torch.tanh((lin('f') + w[p + 'f.b'].to(u.dtype)) / cap))
    S = torch.zeros(H, d, dv, dtype=u.dtype)
    n = torch.zeros(H, d, dtype=u.dtype)
    m = torch.zeros(H, dtype=u.dtype)
    y = torch.zeros(T, H, dv, dtype=u.dtype)
    for t in range(T):
        m_new = torch.maximum(b[t] + m, a[t])
        keep, take = torch.exp(b[t] + m - m_new), torch.exp(a[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        num = torch.einsum('hdv,hd->hv', S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        y[t] = num / den[:, None]
    y = unit_rms(y, eps).reshape(T, H * dv) * w[p + 'norm'].to(u.dtype)
    return (y * torch.sigmoid(lin('g'))) @ w[p + 'o'].to(u.dtype).T


def parallel_mixer(u, w, p, mc, eps):
    return (float(mc['left_scale']) * softmax_window_attention(u, w, p + 'left.', mc['left'])
            + float(mc['right_scale']) * matrix_memory(u, w, p + 'right.', mc['right'], eps))


def unit(h, w, p):
    return relu2(h @ w[p + 'up'].to(h.dtype).T) @ w[p + 'down'].to(h.dtype).T


def route(h, w, p, rc):
    """-> (ids [T, top], weights [T, top]). Router outputs = real experts followed by identity experts; softmax over all of them;
    choice score = probability + correction; only members of the `keep` groups with the largest best-member choice score can be
    chosen; the weights are the chosen probabilities as they are."""
    n_out = w[p + 'router'].shape[0]
    prob = torch.softmax(h @ w[p + 'router'].to(h.dtype).T, -1)
    choice = prob + w[p + 'correction'].to(h.dtype) if (p + 'correction') in w else prob.clone()
    g = rc.get('groups')
    if g and int(g['count']) > 1:
        cnt, keep = int(g['count']), int(g['keep'])
        best = choice.view(-1, cnt, n_out // cnt).max(-1).values
        kept = torch.zeros_like(best, dtype=torch.bool).scatter(1, best.topk(keep, -1).indices, True)
        choice = choice.masked_fill(~kept.repeat_interleave(n_out // cnt, 1), float('-inf'))
    ids = choice.topk(int(rc['top']), -1).indices
    return ids, prob.gather(1, ids)


def moe_ff(h, w, p, fc):
    rc = fc['router']
    n_real = int(rc['experts'])
    ids, wt = route(h, w, p, rc)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, c in zip(ids[t].tolist(), wt[t]):
            out[t] += c * (unit(h[t:t + 1], w, f'{p}e{e}.')[0] if e < n_real else h[t])
    if fc.get('shared'):
        out = out + torch.sigmoid(h @ w[p + 'shared.sg'].to(h.dtype).T) * unit(h, w, p + 'shared.')
    return out


def forward(cfg, weights, tokens, dtype=torch.float32, trace=None):
    """token ids of ONE sequence -> logits [T, vocab]; `trace` (a list) receives the residual stream after every layer"""
    w = {k: v.to(dtype) if v.is_floating_point() else v for k, v in weights.items()}
    eps, r = float(cfg['norm']['eps']), float(cfg.get('residual_mult', 1.0))
    x = w['embed'][torch.as_tensor(tokens, dtype=torch.long)]
    for i, lc in enumerate(cfg['layers']):
        p = f'l{i}.'
        u = token_shift(norm1p(x, w[p + 'norm1'], eps), w[p + 'shift'])
        if lc['type'] == 'parallel':
            y = parallel_mixer(u, w, p + 'mix.', lc['mixer'], eps)
        elif lc['type'] == 'attention':
            y = sigmoid_window_attention(u, w, p + 'mix.', lc['mixer'])
        else:
            raise NotImplementedError(lc['type'])
        x = x + r * norm1p(y, w[p + 'norm1b'], eps)
        fc = lc.get('mlp')
        if fc is not None:
            h = norm1p(x, w[p + 'norm2'], eps)
            y = unit(h, w, p + 'mlp.') if fc['kind'] == 'dense' else moe_ff(h, w, p + 'mlp.', fc)
            x = x + r * norm1p(y, w[p + 'norm2b'], eps)
        if trace is not None:
            trace.append(x.clone())
    return norm1p(x, w['final.norm'], eps) @ w['head'].T
