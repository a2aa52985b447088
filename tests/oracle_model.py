"""A tiny random-init Qwen3.8-shaped model evaluated with the CPU oracle, in the order of the
reference's scalar executor (models/qwen38_27b/src/decoder.rs), plus the loader that gives the same
tensors to the B200 executor. Test infrastructure only."""
import numpy as np

import ctox_llm_b200 as ctox
from ctox_llm_b200 import native as N


def tiny_config(**kw):
    cfg = N.ModelConfig(
        vocab_size=1024, hidden_size=256, intermediate_size=512, num_hidden_layers=4,
        num_attention_heads=4, num_key_value_heads=2, head_dim=64, rotary_dim=16, rope_theta=10_000.0,
        rms_norm_epsilon=1e-6, full_attention_interval=4, linear_num_key_heads=2,
        linear_num_value_heads=4, linear_key_head_dim=128, linear_value_head_dim=128,
        linear_conv_kernel_dim=4, mtp_num_hidden_layers=1, max_context_tokens=256, kv_page_tokens=16,
        kv_dtype=N.F32, max_draft_tokens=4, draft_vocab=0)
    for k, v in kw.items():
        setattr(cfg, k, v)
    return cfg


def bf16_round(x):
    """float32 -> bfloat16 (round to nearest even) -> float32."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    b = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16) << 16
    return b.astype(np.uint32).view(np.float32)


class Matrix:
    def __init__(self, orc, rng, dtype, rows, cols, s_in=None, scale=1.0):
        self.dtype, self.rows, self.cols = dtype, rows, cols
        vals = (rng.standard_normal((rows, cols)) * scale / np.sqrt(cols)).astype(np.float32)
        self.packed = orc.quantize_matrix(dtype, vals)
        self.s_in = s_in if s_in is not None else rng.uniform(0.75, 1.25, cols).astype(np.float16).view(np.uint8)
        self.s_out = rng.uniform(0.75, 1.25, rows).astype(np.float16).view(np.uint8)

    def op(self, orc, x):
        return orc.FusedMatVec(self.dtype, self.packed, self.rows, self.cols, x, s_in=self.s_in,
                               s_out=self.s_out)


class Shard:
    """Rows or columns of a Matrix, as the tensor-parallel executor of one rank loads them."""

    def __init__(self, dtype, packed, rows, cols, s_in, s_out):
        self.dtype, self.packed, self.rows, self.cols, self.s_in, self.s_out = dtype, packed, rows, cols, s_in, s_out


def row_shard(m, ranges):
    sel = np.concatenate([np.arange(a, b) for a, b in ranges])
    packed = np.ascontiguousarray(m.packed.reshape(m.rows, -1)[sel]).reshape(-1)
    s_out = np.ascontiguousarray(m.s_out.reshape(-1, 2)[sel]).reshape(-1)
    return Shard(m.dtype, packed, sel.size, m.cols, m.s_in, s_out)


def col_shard(m, c0, c1):
    blocks = m.cols // 64
    packed = np.ascontiguousarray(m.packed.reshape(m.rows, blocks, -1)[:, c0 // 64:c1 // 64]).reshape(-1)
    s_in = np.ascontiguousarray(m.s_in.reshape(-1, 2)[c0:c1]).reshape(-1)
    return Shard(m.dtype, packed, m.rows, c1 - c0, s_in, m.s_out)


def span(rank, world, total):
    n = total // world
    return rank * n, (rank + 1) * n


def concat(mats):
    """Rows of a fan-out group as one matrix (shared s_in)."""
    m0 = mats[0]
    return ctox.FusedMatVec(m0.dtype, np.concatenate([m.packed for m in mats]),
                            sum(m.rows for m in mats), m0.cols, None, s_in=m0.s_in,
                            s_out=np.concatenate([m.s_out for m in mats]))


class OracleModel:
    def __init__(self, orc, cfg, seed=0):
        self.orc, self.cfg = orc, cfg
        self.kv_bf16 = cfg.kv_dtype == N.BF16  # the cache stores K and V rounded to bfloat16
        rng = np.random.default_rng(seed)
        c = cfg
        H, F = c.hidden_size, c.intermediate_size
        self.qw, self.kvw = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
        self.kw, self.vw = c.linear_num_key_heads * 128, c.linear_num_value_heads * 128
        self.channels = 2 * self.kw + self.vw
        Q4, Q2 = orc.Q4B64, orc.Q2B64
        norm = lambda n: (rng.standard_normal(n) * 0.1).astype(np.float32)
        self.embed = Matrix(orc, rng, Q4, c.vocab_size, H, scale=16.0)
        self.lm_head = Matrix(orc, rng, Q4, c.vocab_size, H, scale=4.0)
        self.final_norm = norm(H)
        self.layers = []
        for l in range(c.num_hidden_layers + c.mtp_num_hidden_layers):
            full = l >= c.num_hidden_layers or (l + 1) % c.full_attention_interval == 0
            L = {"full": full, "in_ln": norm(H), "post_ln": norm(H)}
            sh = rng.uniform(0.75, 1.25, H).astype(np.float16).view(np.uint8)
            if full:
                L["q"] = Matrix(orc, rng, Q4, 2 * self.qw, H, sh, 2.0)
                L["k"] = Matrix(orc, rng, Q4, self.kvw, H, sh, 2.0)
                L["v"] = Matrix(orc, rng, Q4, self.kvw, H, sh, 2.0)
                L["o"] = Matrix(orc, rng, Q4, H, self.qw, None, 2.0)
                L["q_norm"], L["k_norm"] = norm(c.head_dim), norm(c.head_dim)
            else:
                L["qkv"] = Matrix(orc, rng, Q4, self.channels, H, sh, 2.0)
                L["z"] = Matrix(orc, rng, Q4, self.vw, H, sh, 2.0)
                L["a"] = Matrix(orc, rng, Q4, c.linear_num_value_heads, H, sh, 2.0)
                L["b"] = Matrix(orc, rng, Q4, c.linear_num_value_heads, H, sh, 2.0)
                L["out"] = Matrix(orc, rng, Q4, H, self.vw, None, 2.0)
                L["conv_w"] = (rng.standard_normal(self.channels * c.linear_conv_kernel_dim) * 0.5).astype(np.float32)
                L["a_log"] = (rng.standard_normal(c.linear_num_value_heads) * 0.5).astype(np.float32)
                L["dt_bias"] = (rng.standard_normal(c.linear_num_value_heads) * 0.5).astype(np.float32)
                L["lin_norm"] = (1.0 + rng.standard_normal(128) * 0.1).astype(np.float32)
            sg = rng.uniform(0.75, 1.25, H).astype(np.float16).view(np.uint8)
            L["gate"] = Matrix(orc, rng, Q2, F, H, sg, 2.0)
            L["up"] = Matrix(orc, rng, Q2, F, H, sg, 2.0)
            L["down"] = Matrix(orc, rng, Q2, H, F, None, 2.0)
            self.layers.append(L)
        if c.mtp_num_hidden_layers:
            self.mtp_fc = Matrix(orc, rng, Q4, H, 2 * H, None, 2.0)
            self.mtp_norm_e, self.mtp_norm_h, self.mtp_norm = norm(H), norm(H), norm(H)
        self.reset()

    # ---- loading into the device executor
    def load_into(self, ex, rank=0, world=1):
        """Loads the model, or with world > 1 this rank's shard of it: heads, FFN width and
        vocabulary rows [rank/world, (rank+1)/world); norms, embedding and mtp.fc whole."""
        c, G = self.cfg, N.LAYER_GLOBAL
        hd = c.head_dim
        emb = ctox.FusedMatVec(self.embed.dtype, self.embed.packed, self.embed.rows, self.embed.cols, None,
                               s_in=self.embed.s_in, s_out=self.embed.s_out)
        ex.load_matrix(G, N.T_EMBED, emb)
        ex.load_matrix(G, N.T_LM_HEAD, concat([row_shard(self.lm_head, [span(rank, world, c.vocab_size)])]))
        ex.load_vector(G, N.T_FINAL_NORM, self.final_norm)
        q0, q1 = span(rank, world, c.num_attention_heads)
        if c.num_key_value_heads >= world:
            kv0, kv1 = span(rank, world, c.num_key_value_heads)
        else:  # fewer KV heads than ranks: neighbours share one
            kv0 = rank * c.num_key_value_heads // world
            kv1 = kv0 + 1
        lk0, lk1 = span(rank, world, c.linear_num_key_heads)
        lv0, lv1 = span(rank, world, c.linear_num_value_heads)
        f0, f1 = span(rank, world, c.intermediate_size)
        lin_rows = [(lk0 * 128, lk1 * 128), (self.kw + lk0 * 128, self.kw + lk1 * 128),
                    (2 * self.kw + lv0 * 128, 2 * self.kw + lv1 * 128)]
        for l, L in enumerate(self.layers):
            ex.load_vector(l, N.T_INPUT_NORM, L["in_ln"])
            ex.load_vector(l, N.T_POST_NORM, L["post_ln"])
            if L["full"]:
                ex.load_matrix(l, N.T_ATTN_QKV, concat([row_shard(L["q"], [(q0 * 2 * hd, q1 * 2 * hd)]),
                                                        row_shard(L["k"], [(kv0 * hd, kv1 * hd)]),
                                                        row_shard(L["v"], [(kv0 * hd, kv1 * hd)])]))
                ex.load_matrix(l, N.T_ATTN_O, concat([col_shard(L["o"], q0 * hd, q1 * hd)]))
                ex.load_vector(l, N.T_Q_NORM, L["q_norm"])
                ex.load_vector(l, N.T_K_NORM, L["k_norm"])
            else:
                ex.load_matrix(l, N.T_LIN_IN, concat([row_shard(L["qkv"], lin_rows),
                                                      row_shard(L["z"], [(lv0 * 128, lv1 * 128)]),
                                                      row_shard(L["a"], [(lv0, lv1)]),
                                                      row_shard(L["b"], [(lv0, lv1)])]))
                ex.load_matrix(l, N.T_LIN_OUT, concat([col_shard(L["out"], lv0 * 128, lv1 * 128)]))
                kd = c.linear_conv_kernel_dim
                conv = L["conv_w"].reshape(self.channels, kd)
                ex.load_vector(l, N.T_CONV_W, np.concatenate([conv[a:b] for a, b in lin_rows]).reshape(-1))
                ex.load_vector(l, N.T_A_LOG, L["a_log"][lv0:lv1])
                ex.load_vector(l, N.T_DT_BIAS, L["dt_bias"][lv0:lv1])
                ex.load_vector(l, N.T_LIN_NORM, L["lin_norm"])
            ex.load_matrix(l, N.T_MLP_GATE_UP, concat([row_shard(L["gate"], [(f0, f1)]),
                                                       row_shard(L["up"], [(f0, f1)])]))
            ex.load_matrix(l, N.T_MLP_DOWN, concat([col_shard(L["down"], f0, f1)]))
        if c.mtp_num_hidden_layers:
            ex.load_matrix(G, N.T_MTP_FC, concat([self.mtp_fc]))
            ex.load_vector(G, N.T_MTP_NORM_E, self.mtp_norm_e)
            ex.load_vector(G, N.T_MTP_NORM_H, self.mtp_norm_h)
            ex.load_vector(G, N.T_MTP_NORM, self.mtp_norm)

    # ---- scalar evaluation (decoder.rs)
    def reset(self):
        c = self.cfg
        self.position = 0
        self.state = []
        for L in self.layers[: c.num_hidden_layers]:
            if L["full"]:
                self.state.append({"k": [], "v": []})
            else:
                self.state.append({"conv": np.zeros(self.channels * c.linear_conv_kernel_dim, np.float32),
                                   "rec": np.zeros(c.linear_num_value_heads * 128 * 128, np.float32)})

    def proj(self, m, x):
        return self.orc.fused_matvec(m.op(self.orc, x))

    def norm(self, x, w):
        return self.orc.rms_norm_1p_weight(x, 1, x.size, w, self.cfg.rms_norm_epsilon)

    def embedding(self, token):
        e = self.embed
        bb = 34 if e.dtype == self.orc.Q4B64 else 18
        rb = e.cols // 64 * bb
        s_out = np.frombuffer(e.s_out.tobytes(), dtype=np.float16)[token]
        return self.orc.recovered_row(e.dtype, e.packed[token * rb:(token + 1) * rb], e.cols, e.s_in, float(s_out))

    def mlp(self, L, h):  # decoder.rs:636-670
        n = self.norm(h, L["post_ln"])
        act = self.orc.swiglu(self.proj(L["gate"], n), self.proj(L["up"], n))
        return h + self.proj(L["down"], act)

    def full_attention(self, L, h, rope_pos, st):  # decoder.rs:687-800
        c, orc = self.cfg, self.orc
        n = self.norm(h, L["in_ln"])
        qg = self.proj(L["q"], n).reshape(c.num_attention_heads, 2, c.head_dim)
        query, gate = qg[:, 0, :].reshape(-1), qg[:, 1, :].reshape(-1)
        key, value = self.proj(L["k"], n), self.proj(L["v"], n)
        query = orc.rms_norm_1p_weight(query, c.num_attention_heads, c.head_dim, L["q_norm"], c.rms_norm_epsilon)
        key = orc.rms_norm_1p_weight(key, c.num_key_value_heads, c.head_dim, L["k_norm"], c.rms_norm_epsilon)
        query, key = orc.apply_partial_rope(query, key, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
                                            c.rotary_dim, rope_pos, c.rope_theta)
        if self.kv_bf16:
            key, value = bf16_round(key), bf16_round(value)
        st["k"].append(key)
        st["v"].append(value)
        T = len(st["k"])
        K = np.stack(st["k"]).reshape(T, c.num_key_value_heads, c.head_dim).transpose(1, 0, 2)
        V = np.stack(st["v"]).reshape(T, c.num_key_value_heads, c.head_dim).transpose(1, 0, 2)
        att = orc.grouped_query_attention(query, K, V, c.num_attention_heads, c.num_key_value_heads, 1, T,
                                          c.head_dim, T - 1)
        att = orc.sigmoid_gate(att, gate)
        return h + self.proj(L["o"], att)

    def linear_attention(self, L, h, st):  # decoder.rs:806-938
        c, orc = self.cfg, self.orc
        n = self.norm(h, L["in_ln"])
        mixed, z = self.proj(L["qkv"], n), self.proj(L["z"], n)
        a, b = self.proj(L["a"], n), self.proj(L["b"], n)
        conv, st["conv"] = orc.causal_conv_silu_update(mixed, st["conv"], L["conv_w"], self.channels,
                                                       c.linear_conv_kernel_dim)
        rep = c.linear_num_value_heads // c.linear_num_key_heads
        q = np.repeat(conv[: self.kw].reshape(-1, 128), rep, axis=0).reshape(-1)
        k = np.repeat(conv[self.kw: 2 * self.kw].reshape(-1, 128), rep, axis=0).reshape(-1)
        v = conv[2 * self.kw:]
        g, beta = orc.gated_delta_prepare(a, b, L["a_log"], L["dt_bias"])
        core, st["rec"] = orc.recurrent_gated_delta_step(q, k, v, g, beta, st["rec"], c.linear_num_value_heads,
                                                         128, 128)
        core = orc.rms_norm_gated(core, z, c.linear_num_value_heads, 128, L["lin_norm"], c.rms_norm_epsilon)
        return h + self.proj(L["out"], core)

    def decode_target_step(self, token):  # decoder.rs:956-998
        h = self.embedding(token)
        for l in range(self.cfg.num_hidden_layers):
            L, st = self.layers[l], self.state[l]
            h = self.full_attention(L, h, self.position, st) if L["full"] else self.linear_attention(L, h, st)
            h = self.mlp(L, h)
        final_hidden = self.norm(h, self.final_norm)
        logits = self.proj(self.lm_head, final_hidden)
        self.position += 1
        return final_hidden, logits

    def greedy(self, prompt, n_new):
        """Consumes the prompt, then generates n_new tokens greedily (sampler.rs:76-82)."""
        self.reset()
        out, logits_trace = [], []
        for t in prompt[:-1]:
            self.decode_target_step(int(t))
        tok = int(prompt[-1])
        for _ in range(n_new):
            fh, logits = self.decode_target_step(tok)
            tok = self.orc.greedy_token(logits)
            out.append(tok)
            logits_trace.append(logits)
        return out, logits_trace, fh
