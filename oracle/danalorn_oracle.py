"""Plain, slow restatement of the Danalorn decoder (torch on the CPU, float32 or float64), one function per mechanism.

It shares no code with the CUDA path: the tests build small random checkpoints, run both and compare. A sequence is processed
whole, token loops where the design is recurrent, no cache and no state object.

Notation: x residual stream [T, W]; N(v; g) = v / sqrt(mean(v^2) + eps) * g. The stream starts as
    x_t = E[tok_t] * s + B[(tok_(t-1) * m_p + tok_t * m_c) mod n]        (B's last row, number n, for the first token)
and a layer is
    x <- x + N(mixer(N(x; g1)); g1b);   x <- x + N(ff(N(x; g2)); g2b)
Mixers:
  'latent_attention'  queries through a normed low-rank vector; one normed latent vector and one rotated key part per token serve
                      all heads (keys and values are up-projections of the latent vector); neighbouring numbers rotate as pairs;
                      sliding window; a learned per-head sink in the softmax denominator. A layer with `kv_from` reads the latent
                      vectors and rotated key parts another layer made, through up-projections of its own;
  'attention'         grouped-query attention with projection biases, per-head query/key RMS norm, no rotation, queries that grow
                      with the logarithm of their position in steps, a linear distance bias per head, one added to the softmax
                      denominator, and an element-wise sigmoid gate on the concatenated heads;
  'gla'               gated linear attention: per head a matrix state with one decay per key channel and token (from a low-rank
                      projection), read out by the query, normed per head and gated by silu.
Feed-forward: W_down relu(W_up h)^2. cfg is the parsed config.json (a dict), w the tensor dict of the checkpoint.
"""
import torch


def rms_norm(v, g, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * g


def embed(tokens, w, ec, dtype):
    """scaled token rows plus the row of a hashed (previous, current) pair; the first token takes the table's last row"""
    tok = [int(t) for t in tokens]
    x = w['embed'][torch.tensor(tok)].to(dtype) * float(ec.get('scale', 1.0))
    bg = ec.get('bigram')
    if bg:
        n, mp, mc = int(bg['buckets']), int(bg['mul_prev']), int(bg['mul_cur'])
        rows = [n if t == 0 else (tok[t - 1] * mp + tok[t] * mc) % n for t in range(len(tok))]
        x = x + w['bigram'][torch.tensor(rows)].to(dtype)
    return x


def rotate_pairs(v, pos, rot):
    """v [T, heads, d]: numbers 2i and 2i + 1 (2i + 1 < dims) turn together by pos * base^(-2i/dims); the rest stays"""
    dims = int(rot['dims'])
    f = float(rot['base']) ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
    ang = pos.to(v.dtype)[:, None] * f.to(v.dtype)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out = v.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def causal_window(T, size):
    """[T, T] bool: query i sees key j when 0 <= i - j and (size == 0 or i - j < size)"""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) if size else torch.ones(T, T, dtype=torch.bool))


def softmax_with_sink(s, vis, sink):
    """rows of s over the visible keys; exp(sink) joins the denominator only"""
    s = s.masked_fill(~vis, float('-inf'))
    m = torch.maximum(s.max(-1, keepdim=True).values, torch.as_tensor(sink, dtype=s.dtype))
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(torch.as_tensor(sink, dtype=s.dtype) - m))


def latent_kv(h, w, p, mc, eps):
    """-> (normed latent vectors [T, kv_rank], rotated shared key parts [T, rot_dim]) of the layer whose tensors start with p"""
    T = h.shape[0]
    R, dr = int(mc['kv_rank']), int(mc['rot_dim'])
    ckv = h @ w[p + 'dkv'].to(h.dtype).T
    c = rms_norm(ckv[:, :R], w[p + 'dkv.norm'].to(h.dtype), eps)
    kr = rotate_pairs(ckv[:, R:R + dr].reshape(T, 1, dr), torch.arange(T), mc['rot'])[:, 0]
    return c, kr


def latent_attention(h, w, p, mc, eps, kv):
    """kv = (c, kr) as latent_kv returns them: this layer's own, or the source layer's when the mixer has `kv_from`"""
    T = h.shape[0]
    H, d, dr, dv, R = int(mc['heads']), int(mc['dim']), int(mc['rot_dim']), int(mc['vdim']), int(mc['kv_rank'])
    c, kr = kv
    cq = rms_norm(h @ w[p + 'dq'].to(h.dtype).T, w[p + 'dq.norm'].to(h.dtype), eps)
    q = (cq @ w[p + 'uq'].to(h.dtype).T).view(T, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], torch.arange(T), mc['rot'])
    k_plain = (c @ w[p + 'uk'].to(h.dtype).T).view(T, H, d)
    v = (c @ w[p + 'uv'].to(h.dtype).T).view(T, H, dv)
    vis = causal_window(T, int((mc.get('mask') or {}).get('size', 0) or 0))
    sink = w[p + 'sink'].to(h.dtype)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        s = (q_plain[:, hh] @ k_plain[:, hh].T + q_rot[:, hh] @ kr.T) * float(mc['scale'])
        out[:, hh] = softmax_with_sink(s, vis, sink[hh]) @ v[:, hh]
    return out.reshape(T, H * dv) @ w[p + 'o'].to(h.dtype).T


def biased_attention(h, w, p, mc, eps):
    T = h.shape[0]
    H, G, d, dv = int(mc['heads']), int(mc.get('kv_heads', mc['heads'])), int(mc['dim']), int(mc.get('vdim', mc['dim']))
    lin = lambda n: h @ w[p + n].to(h.dtype).T + w[p + n + '.b'].to(h.dtype)
    q = rms_norm(lin('q').view(T, H, d), w[p + 'q.norm'].to(h.dtype), eps)
    k = rms_norm(lin('k').view(T, G, d), w[p + 'k.norm'].to(h.dtype), eps)
    v = lin('v').view(T, G, dv)
    qt = mc.get('q_temp')
    if qt:
        pos = torch.arange(T)
        steps = torch.div(pos + 1, int(qt['every']), rounding_mode='floor')
        q = q * (1.0 + float(qt['coef']) * torch.log(steps.to(h.dtype) + 1.0))[:, None, None]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    vis = j <= i
    dist = (i - j).to(h.dtype)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        slope = 2.0 ** (-8.0 * (hh + 1) / H)
        s = (q[:, hh] @ k[:, g].T) * float(mc['scale']) - slope * dist
        out[:, hh] = softmax_with_sink(s, vis, 0.0) @ v[:, g]
    gate = torch.sigmoid(h @ w[p + 'g'].to(h.dtype).T)
    return (out.reshape(T, H * dv) * gate) @ w[p + 'o'].to(h.dtype).T


def gated_linear_attention(h, w, p, mc, eps):
    """token by token. Per head a state S [d, dv] that starts at zero: S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t,
    a_t = sigmoid(z_t)^(1/tau) per key channel"""
    T = h.shape[0]
    H, d, dv, tau = int(mc['heads']), int(mc['dim']), int(mc.get('vdim', mc['dim'])), float(mc['tau'])
    lin = lambda n: h @ w[p + n].to(h.dtype).T
    q = lin('q').view(T, H, d) * d ** -0.5
    k = lin('k').view(T, H, d)
    v = lin('v').view(T, H, dv)
    z = lin('a1') @ w[p + 'a2'].to(h.dtype).T + w[p + 'a2.b'].to(h.dtype)
    a = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum('hdv,hd->hv', S, q[t])
    o = rms_norm(o, w[p + 'norm'].to(h.dtype), eps).reshape(T, H * dv)
    return (o * torch.nn.functional.silu(lin('g'))) @ w[p + 'o'].to(h.dtype).T


def dense_ff(h, w, p):
    return torch.relu(h @ w[p + 'up'].to(h.dtype).T) ** 2 @ w[p + 'down'].to(h.dtype).T


def forward(cfg, weights, tokens, dtype=torch.float32, trace=None):
    """token ids of ONE sequence -> logits [T, vocab]; `trace` (a list) receives the residual stream after every layer"""
    w = {k: v.to(dtype) if v.is_floating_point() else v for k, v in weights.items()}
    eps = float(cfg['norm']['eps'])
    x = embed(tokens, w, cfg.get('embedding') or {}, dtype)
    kv = {}
    for i, lc in enumerate(cfg['layers']):
        p, mc = f'l{i}.', lc['mixer']
        h = rms_norm(x, w[p + 'norm1'], eps)
        if lc['type'] == 'latent_attention':
            src = mc.get('kv_from')
            if src is None:
                kv[i] = latent_kv(h, w, p + 'mix.', mc, eps)
            y = latent_attention(h, w, p + 'mix.', mc, eps, kv[i if src is None else int(src)])
        elif lc['type'] == 'attention':
            y = biased_attention(h, w, p + 'mix.', mc, eps)
        elif lc['type'] == 'gla':
            y = gated_linear_attention(h, w, p + 'mix.', mc, eps)
        else:
            raise NotImplementedError(lc['type'])
        x = x + rms_norm(y, w[p + 'norm1b'], eps)
        if lc.get('mlp') is not None:
            if lc['mlp']['kind'] != 'dense':
                raise NotImplementedError(lc['mlp']['kind'])
            x = x + rms_norm(dense_ff(rms_norm(x, w[p + 'norm2'], eps), w, p + 'mlp.'), w[p + 'norm2b'], eps)
        if trace is not None:
            trace.append(x.clone())
    return rms_norm(x, w['final.norm'], eps) @ w['head'].T
