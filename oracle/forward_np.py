"""TEST INFRASTRUCTURE - not part of the product.

A second, independent restatement of the reference's scalar CPU forward for one token of the hybrid target
(crates/qwen-llm/src/forward.rs: driver :96-161 / :173-220, ffn :725-747, ffn_moe :749-824, attn_step :834-932,
gdn_step :940-1107, KvCache :1133-1240, primitives :1256-1371), written in numpy against the reference text, not
against oracle/forward.hpp.  Weights are decoded by the `gguf` package's numpy dequantisers, not by oracle/quants.hpp,
so agreement between this module and the C++ oracle checks both the forward restatement and the block decoders by
two routes.  Matrix products are numpy's (another summation order than the reference's sequential loops), hence
agreement to a tolerance, not bit for bit.  Only tests import this file.
"""
import numpy as np

F32, F16, Q8_0, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 8, 12, 13, 14, 30
RMS_EPS = np.float32(1e-6)


def decode(dtype, raw, n_elements):
    """ggml bytes -> f32, through the gguf package for the block formats."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    if dtype == F32:
        return raw.view(np.float32)[:n_elements].copy()
    if dtype == F16:
        return raw.view(np.float16)[:n_elements].astype(np.float32)
    if dtype == BF16:
        return (raw.view(np.uint16)[:n_elements].astype(np.uint32) << 16).view(np.float32)
    import gguf
    qt = {Q8_0: gguf.GGMLQuantizationType.Q8_0, Q4_K: gguf.GGMLQuantizationType.Q4_K, Q5_K: gguf.GGMLQuantizationType.Q5_K,
          Q6_K: gguf.GGMLQuantizationType.Q6_K}[dtype]
    return np.asarray(gguf.quants.dequantize(raw, qt), dtype=np.float32).reshape(-1)[:n_elements]


def rms_norm(x, w, eps):                       # forward.rs:1256-1264
    mean_sq = np.float32(np.sum(x * x, dtype=np.float32) / np.float32(x.size))
    return (x * (np.float32(1.0) / np.sqrt(mean_sq + eps)) * w).astype(np.float32)


def l2_norm(x, eps):                           # forward.rs:1269-1275: x / max(||x||, eps)
    return (x * (np.float32(1.0) / max(np.sqrt(np.sum(x * x, dtype=np.float32)), eps))).astype(np.float32)


def silu(x):                                   # forward.rs:1278-1280
    return (x / (np.float32(1.0) + np.exp(-x))).astype(np.float32)


def sigmoid(x):                                # forward.rs:1283-1285
    return (np.float32(1.0) / (np.float32(1.0) + np.exp(-x))).astype(np.float32)


def softplus(x):                               # forward.rs:1288-1296: x above 20, exp(x) below -20
    x = np.asarray(x, dtype=np.float32)
    mid = np.log1p(np.exp(np.clip(x, -20, 20))).astype(np.float32)
    return np.where(x > 20, x, np.where(x < -20, np.exp(np.minimum(x, 0)), mid)).astype(np.float32)


def softmax(x):                                # forward.rs:1298-1308
    e = np.exp(x - np.max(x)).astype(np.float32)
    return (e * (np.float32(1.0) / np.sum(e, dtype=np.float32))).astype(np.float32)


def rope(buf, n_heads, head_dim, n_rot, position, theta):   # forward.rs:1343-1371, NeoX pairs (i, i + n_rot / 2)
    out = buf.reshape(n_heads, head_dim).copy()
    half = n_rot // 2
    i = np.arange(half, dtype=np.float32)
    freq = np.float32(position) / np.power(np.float32(theta), (2 * i) / np.float32(n_rot), dtype=np.float32)
    s, c = np.sin(freq).astype(np.float32), np.cos(freq).astype(np.float32)
    a, b = out[:, :half].copy(), out[:, half:2 * half].copy()
    out[:, :half] = a * c - b * s
    out[:, half:2 * half] = a * s + b * c
    return out.reshape(-1)


class State:
    def __init__(self, model, kv_f16):
        a = model.a
        conv_dim = (2 * a["gdn_n_k_heads"] + a["gdn_n_v_heads"]) * a["gdn_head_dim"]
        self.conv = [np.zeros((a["gdn_conv_kernel"] - 1, conv_dim), dtype=np.float32) for _ in range(model.n_gdn)]
        self.ssm = [np.zeros((a["gdn_n_v_heads"], a["gdn_head_dim"], a["gdn_head_dim"]), dtype=np.float32) for _ in range(model.n_gdn)]
        self.k = {il: [] for il in model.attn_layers}   # per attention layer: list of [n_kv, hd] rows by position
        self.v = {il: [] for il in model.attn_layers}
        self.kv_f16 = kv_f16
        self.last_route = None


class Model:
    def __init__(self, arch, tensors):
        """arch: any object with the dfl_arch fields; tensors: [(name, dtype, shape [fastest first], bytes)]."""
        fields = ["n_layer", "hidden_size", "intermediate_size", "vocab_size", "full_attention_interval", "n_q_heads", "n_kv_heads",
                  "attn_head_dim", "rope_theta", "partial_rotary_factor", "gdn_n_v_heads", "gdn_n_k_heads", "gdn_head_dim",
                  "gdn_conv_kernel", "expert_count", "expert_used_count", "expert_feed_forward_length",
                  "expert_shared_feed_forward_length"]
        self.a = {f: getattr(arch, f) for f in fields}
        self.t = {}
        for name, dtype, shape, raw in tensors:
            n = int(np.prod(shape))
            self.t[name] = decode(dtype, raw, n).reshape(tuple(reversed(shape)))   # ggml: first extent fastest
        iv = max(self.a["full_attention_interval"], 1)
        self.attn_layers = [il for il in range(self.a["n_layer"]) if il % iv == iv - 1]
        self.n_gdn = self.a["n_layer"] - len(self.attn_layers)

    def new_state(self, kv_f16=False):
        return State(self, kv_f16)

    def w(self, name):
        return self.t[name]

    # ---- blocks ---------------------------------------------------------------------------
    def ffn(self, il, x, st):
        b = f"blk.{il}."
        a = self.a
        if a["expert_count"] > 0:                                  # forward.rs:749-824
            probs = softmax(self.w(b + "ffn_gate_inp.weight") @ x)
            k = min(a["expert_used_count"], a["expert_count"])
            order = sorted(range(probs.size), key=lambda e: (-float(probs[e]), e))[:k]   # by probability, then index
            st.last_route = list(order)
            wsum = max(np.float32(sum(np.float32(probs[e]) for e in order)), np.float32(2.0 ** -14))
            out = np.zeros(a["hidden_size"], dtype=np.float32)
            ge, ue, de = self.w(b + "ffn_gate_exps.weight"), self.w(b + "ffn_up_exps.weight"), self.w(b + "ffn_down_exps.weight")
            for e in order:
                hid = silu(ge[e] @ x) * (ue[e] @ x)
                out += (probs[e] / wsum) * (de[e] @ hid)
            gate = sigmoid(np.float32(np.dot(x, self.w(b + "ffn_gate_inp_shexp.weight").reshape(-1))))
            hid = silu(self.w(b + "ffn_gate_shexp.weight") @ x) * (self.w(b + "ffn_up_shexp.weight") @ x)
            return (out + gate * (self.w(b + "ffn_down_shexp.weight") @ hid)).astype(np.float32)
        hid = silu(self.w(b + "ffn_gate.weight") @ x) * (self.w(b + "ffn_up.weight") @ x)   # forward.rs:725-747
        return (self.w(b + "ffn_down.weight") @ hid).astype(np.float32)

    def attn(self, il, x, position, st):                         # forward.rs:834-932
        b = f"blk.{il}."
        a = self.a
        hd, n_q, n_kv = a["attn_head_dim"], a["n_q_heads"], a["n_kv_heads"]
        n_rot = int(np.float32(hd) * np.float32(a["partial_rotary_factor"]))
        qf = (self.w(b + "attn_q.weight") @ x).reshape(n_q, 2, hd)   # per head: q then gate
        q, gate = qf[:, 0, :].copy(), qf[:, 1, :].copy()
        q = np.stack([rms_norm(q[h], self.w(b + "attn_q_norm.weight"), RMS_EPS) for h in range(n_q)])
        k = (self.w(b + "attn_k.weight") @ x).reshape(n_kv, hd)
        v = (self.w(b + "attn_v.weight") @ x).reshape(n_kv, hd).astype(np.float32)
        k = np.stack([rms_norm(k[h], self.w(b + "attn_k_norm.weight"), RMS_EPS) for h in range(n_kv)])
        q = rope(q.reshape(-1), n_q, hd, n_rot, position, a["rope_theta"]).reshape(n_q, hd)
        k = rope(k.reshape(-1), n_kv, hd, n_rot, position, a["rope_theta"]).reshape(n_kv, hd)
        if st.kv_f16:
            k, v = k.astype(np.float16).astype(np.float32), v.astype(np.float16).astype(np.float32)
        assert len(st.k[il]) == position, "positions must be appended in order"
        st.k[il].append(k)
        st.v[il].append(v)
        K, V = np.stack(st.k[il]), np.stack(st.v[il])             # [n_pos, n_kv, hd]
        group = n_q // n_kv
        scale = np.float32(1.0) / np.sqrt(np.float32(hd))
        out = np.zeros((n_q, hd), dtype=np.float32)
        for h in range(n_q):
            p = softmax((K[:, h // group, :] @ q[h]) * scale)
            out[h] = p @ V[:, h // group, :]
        out = out * sigmoid(gate)
        return (self.w(b + "attn_output.weight") @ out.reshape(-1)).astype(np.float32)

    def gdn(self, gi, il, x, st):                                 # forward.rs:940-1107
        b = f"blk.{il}."
        a = self.a
        n_v, n_k, hd, kk = a["gdn_n_v_heads"], a["gdn_n_k_heads"], a["gdn_head_dim"], a["gdn_conv_kernel"]
        qkv = (self.w(b + "attn_qkv.weight") @ x).astype(np.float32)
        z = (self.w(b + "attn_gate.weight") @ x).reshape(n_v, hd)
        beta = sigmoid(self.w(b + "ssm_beta.weight") @ x)
        alpha = (self.w(b + "ssm_alpha.weight") @ x) + self.w(b + "ssm_dt.bias").reshape(-1)
        g = softplus(alpha) * self.w(b + "ssm_a").reshape(-1)
        conv_w = self.w(b + "ssm_conv1d.weight")                   # [conv_dim, kernel]
        window = np.concatenate([st.conv[gi], qkv[None, :]], axis=0)   # kernel rows, oldest first
        conv_out = silu(np.einsum("ck,kc->c", conv_w, window).astype(np.float32))
        st.conv[gi] = window[1:].copy()
        qd = n_k * hd
        q = np.stack([l2_norm(conv_out[h * hd:(h + 1) * hd], RMS_EPS) for h in range(n_k)])
        k = np.stack([l2_norm(conv_out[qd + h * hd:qd + (h + 1) * hd], RMS_EPS) for h in range(n_k)])
        v = conv_out[2 * qd:].reshape(n_v, hd)
        o = np.zeros((n_v, hd), dtype=np.float32)
        S = st.ssm[gi]
        for h in range(n_v):
            hk = h % n_k
            gh, bh = np.exp(g[h]).astype(np.float32), beta[h]
            sk = S[h] @ k[hk]                                     # S[dv, dk] k[dk], state before the decay
            coeff = bh * (v[h] - gh * sk)
            S[h] = gh * S[h] + np.outer(coeff, k[hk])
            o[h] = S[h] @ q[hk]
        nw = self.w(b + "ssm_norm.weight").reshape(-1)
        y = np.stack([rms_norm(o[h], nw, RMS_EPS * np.float32(hd)) * silu(z[h]) for h in range(n_v)])
        return (self.w(b + "ssm_out.weight") @ y.reshape(-1)).astype(np.float32)

    # ---- driver: forward.rs:96-161 and :173-220 --------------------------------------------
    def single_token(self, st, token, position, layer_ids=()):
        a = self.a
        assert 0 <= token < a["vocab_size"]
        x = self.w("token_embd.weight")[token].astype(np.float32).copy()
        captured = np.zeros((len(layer_ids), a["hidden_size"]), dtype=np.float32)
        gi = 0
        for il in range(a["n_layer"]):
            b = f"blk.{il}."
            cur = rms_norm(x, self.w(b + "attn_norm.weight").reshape(-1), RMS_EPS)
            if il in self.attn_layers:
                cur = self.attn(il, cur, position, st)
            else:
                cur = self.gdn(gi, il, cur, st)
                gi += 1
            x = x + cur
            post = rms_norm(x, self.w(b + "post_attention_norm.weight").reshape(-1), RMS_EPS)
            x = (x + self.ffn(il, post, st)).astype(np.float32)
            for j, lid in enumerate(layer_ids):
                if lid == il:
                    captured[j] = x
        normed = rms_norm(x, self.w("output_norm.weight").reshape(-1), RMS_EPS)
        head = self.t.get("output.weight", self.t["token_embd.weight"])
        return (head @ normed).astype(np.float32), captured


class Drafter:
    """The DFlash drafter's forward for one block (forward.rs:380-662): cross-context projection + norm, noise
    embedding from the target, per layer bidirectional / sliding-window attention over [context ; noise] keys with
    full NeoX RoPE, SwiGLU FFN, then the target's lm_head."""

    def __init__(self, cfg, tensors):
        fields = ["n_layer", "hidden_size", "intermediate_size", "n_q_heads", "n_kv_heads", "head_dim", "rope_theta", "rms_norm_eps",
                  "causal", "swa_window", "block_size", "n_target_layers"]
        self.c = {f: getattr(cfg, f) for f in fields}
        self.is_swa = [bool(cfg.layer_is_swa[i]) for i in range(cfg.n_layer)]
        self.t = {}
        for name, dtype, shape, raw in tensors:
            if name.startswith("selector_"):
                continue
            self.t[name] = decode(dtype, raw, int(np.prod(shape))).reshape(tuple(reversed(shape)))

    def draft(self, target: "Model", noise_ids, ctx_stacked, pos_ctx, noise_start):
        c, w = self.c, self.t
        eps = np.float32(c["rms_norm_eps"])
        H, hd, n_q, n_kv = c["hidden_size"], c["head_dim"], c["n_q_heads"], c["n_kv_heads"]
        group = n_q // n_kv
        n = len(noise_ids)
        pos_ctx = np.asarray(pos_ctx, dtype=np.int64)
        n_ctx = pos_ctx.size
        ctx = np.asarray(ctx_stacked, dtype=np.float32).reshape(n_ctx, -1)
        ctx_h = np.stack([rms_norm(w["dflash_fc.weight"] @ ctx[i], w["dflash_hidden_norm.weight"].reshape(-1), eps) for i in range(n_ctx)]) \
            if n_ctx else np.zeros((0, H), dtype=np.float32)
        x = np.stack([target.w("token_embd.weight")[int(t)].astype(np.float32) for t in noise_ids])
        q_pos = noise_start + np.arange(n, dtype=np.int64)
        k_pos = np.concatenate([pos_ctx, q_pos])
        scale = np.float32(1.0) / np.sqrt(np.float32(hd))
        for il in range(c["n_layer"]):
            b = f"blk.{il}."
            nn = np.stack([rms_norm(x[i], w[b + "attn_norm.weight"].reshape(-1), eps) for i in range(n)])
            rows = np.concatenate([ctx_h, nn])                      # keys / values: context first, noise second
            q = (nn @ w[b + "attn_q.weight"].T).reshape(n, n_q, hd)
            k = (rows @ w[b + "attn_k.weight"].T).reshape(-1, n_kv, hd)
            v = (rows @ w[b + "attn_v.weight"].T).reshape(-1, n_kv, hd).astype(np.float32)
            qn, kn = w[b + "attn_q_norm.weight"].reshape(-1), w[b + "attn_k_norm.weight"].reshape(-1)
            q = np.stack([rope(np.stack([rms_norm(q[i, h], qn, eps) for h in range(n_q)]).reshape(-1), n_q, hd, hd, int(q_pos[i]), c["rope_theta"])
                          for i in range(n)]).reshape(n, n_q, hd)
            k = np.stack([rope(np.stack([rms_norm(k[j, h], kn, eps) for h in range(n_kv)]).reshape(-1), n_kv, hd, hd, int(k_pos[j]), c["rope_theta"])
                          for j in range(k.shape[0])]).reshape(-1, n_kv, hd)
            out = np.zeros((n, n_q, hd), dtype=np.float32)
            for i in range(n):
                allowed = np.ones(k_pos.size, dtype=bool)
                if c["causal"]:
                    allowed &= k_pos <= q_pos[i]
                if self.is_swa[il] and c["swa_window"] != 0:
                    allowed &= np.abs(k_pos - q_pos[i]) < c["swa_window"]
                for h in range(n_q):
                    s = np.where(allowed, (k[:, h // group, :] @ q[i, h]) * scale, -np.inf).astype(np.float32)
                    out[i, h] = softmax(s) @ v[:, h // group, :]
            x = x + out.reshape(n, -1) @ w[b + "attn_output.weight"].T
            h2 = np.stack([rms_norm(x[i], w[b + "post_attention_norm.weight"].reshape(-1), eps) for i in range(n)])
            x = (x + (silu(h2 @ w[b + "ffn_gate.weight"].T) * (h2 @ w[b + "ffn_up.weight"].T)) @ w[b + "ffn_down.weight"].T).astype(np.float32)
        normed = np.stack([rms_norm(x[i], w["output_norm.weight"].reshape(-1), eps) for i in range(n)])
        head = target.t.get("output.weight", target.t["token_embd.weight"])
        return (normed @ head.T).astype(np.float32), normed
