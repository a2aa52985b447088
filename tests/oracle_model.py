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

    @classmethod
    def random_packed(cls, orc, rng, dtype, rows, cols, s_in=None):
        """Random canonical blocks drawn directly as bytes (codes uniform, f16 block scales
        exp(N(-4, 0.5))): what the benchmark's synthetic model holds, cheap enough for full-width
        matrices. One random chunk of a million blocks is repeated with a block-dependent byte added."""
        m = cls.__new__(cls)
        m.dtype, m.rows, m.cols = dtype, rows, cols
        bb = 34 if dtype == orc.Q4B64 else 18
        blocks = rows * (cols // 64)
        chunk = min(blocks, 1 << 20)
        base = np.frombuffer(rng.bytes(chunk * bb), dtype=np.uint8).reshape(chunk, bb)
        out = np.tile(base, (-(-blocks // chunk), 1))[:blocks].copy()
        out += ((np.arange(blocks, dtype=np.uint64) // chunk * 37) & 0xff).astype(np.uint8)[:, None]
        scales = np.exp(rng.standard_normal(blocks, dtype=np.float32) * 0.5 - 4.0).astype(np.float16)
        out.view(np.uint16).reshape(blocks, bb // 2)[:, 0] = scales.view(np.uint16)
        m.packed = out.reshape(-1)
        m.s_in = s_in if s_in is not None else rng.uniform(0.75, 1.25, cols).astype(np.float16).view(np.uint8)
        m.s_out = rng.uniform(0.75, 1.25, rows).astype(np.float16).view(np.uint8)
        return m

    @classmethod
    def constant(cls, orc, dtype, rows, cols, value):
        """Every weight equal to `value`, unit recovery scales: the matrices of the reference's
        decoder fixture (decoder.rs:1505-1530 `recovered_matrix`)."""
        m = cls.__new__(cls)
        m.dtype, m.rows, m.cols = dtype, rows, cols
        m.packed = orc.quantize_matrix(dtype, np.full((rows, cols), value, dtype=np.float32))
        m.s_in = np.ones(cols, dtype=np.float16).view(np.uint8)
        m.s_out = np.ones(rows, dtype=np.float16).view(np.uint8)
        return m

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
    def __init__(self, orc, cfg, seed=0, loud_tokens=(), packed_random=False, threads=1, tied_head=False):
        """loud_tokens: lm_head rows whose output scale is raised so far above the rest that the
        greedy token is nearly always one of them; target and MTP drafts then agree often enough
        for natural (unforced) acceptance to be exercised on a random-init model."""
        self.orc, self.cfg = orc, cfg
        self.threads = threads  # host threads of the oracle's matvec (rows split; same arithmetic per row)
        self.kv_bf16 = cfg.kv_dtype == N.BF16  # the cache stores K and V rounded to bfloat16
        rng = np.random.default_rng(seed)
        if packed_random:  # full-width models: draw the packed bytes directly instead of quantising floats
            make = lambda orc_, rng_, dtype, rows, cols, s_in=None, scale=1.0: Matrix.random_packed(
                orc_, rng_, dtype, rows, cols, s_in)
        else:
            make = Matrix
        c = cfg
        H, F = c.hidden_size, c.intermediate_size
        self.qw, self.kvw = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
        self.kd, self.vd = c.linear_key_head_dim, c.linear_value_head_dim
        self.kw, self.vw = c.linear_num_key_heads * self.kd, c.linear_num_value_heads * self.vd
        self.channels = 2 * self.kw + self.vw
        Q4, Q2 = orc.Q4B64, orc.Q2B64
        norm = lambda n: (rng.standard_normal(n) * 0.1).astype(np.float32)
        self.embed = make(orc, rng, Q4, c.vocab_size, H, scale=16.0)
        self.lm_head = self.embed if tied_head else make(orc, rng, Q4, c.vocab_size, H, scale=4.0)
        if len(loud_tokens):
            so = self.lm_head.s_out.view(np.float16).copy()
            so[list(loud_tokens)] = np.float16(8.0)
            self.lm_head.s_out = so.view(np.uint8)
        self.final_norm = norm(H)
        self.layers = []
        for l in range(c.num_hidden_layers + c.mtp_num_hidden_layers):
            full = l >= c.num_hidden_layers or (l + 1) % c.full_attention_interval == 0
            L = {"full": full, "in_ln": norm(H), "post_ln": norm(H)}
            sh = rng.uniform(0.75, 1.25, H).astype(np.float16).view(np.uint8)
            if full:
                L["q"] = make(orc, rng, Q4, 2 * self.qw, H, sh, 2.0)
                L["k"] = make(orc, rng, Q4, self.kvw, H, sh, 2.0)
                L["v"] = make(orc, rng, Q4, self.kvw, H, sh, 2.0)
                L["o"] = make(orc, rng, Q4, H, self.qw, None, 2.0)
                L["q_norm"], L["k_norm"] = norm(c.head_dim), norm(c.head_dim)
            else:
                L["qkv"] = make(orc, rng, Q4, self.channels, H, sh, 2.0)
                L["z"] = make(orc, rng, Q4, self.vw, H, sh, 2.0)
                L["a"] = make(orc, rng, Q4, c.linear_num_value_heads, H, sh, 2.0)
                L["b"] = make(orc, rng, Q4, c.linear_num_value_heads, H, sh, 2.0)
                L["out"] = make(orc, rng, Q4, H, self.vw, None, 2.0)
                L["conv_w"] = (rng.standard_normal(self.channels * c.linear_conv_kernel_dim) * 0.5).astype(np.float32)
                L["a_log"] = (rng.standard_normal(c.linear_num_value_heads) * 0.5).astype(np.float32)
                L["dt_bias"] = (rng.standard_normal(c.linear_num_value_heads) * 0.5).astype(np.float32)
                L["lin_norm"] = (1.0 + rng.standard_normal(self.vd) * 0.1).astype(np.float32)
            sg = rng.uniform(0.75, 1.25, H).astype(np.float16).view(np.uint8)
            L["gate"] = make(orc, rng, Q2, F, H, sg, 2.0)
            L["up"] = make(orc, rng, Q2, F, H, sg, 2.0)
            L["down"] = make(orc, rng, Q2, H, F, None, 2.0)
            self.layers.append(L)
        if c.mtp_num_hidden_layers:
            self.mtp_fc = make(orc, rng, Q4, H, 2 * H, None, 2.0)
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

    # ---- the model as a CTOXQ container (tensor names of tensor_contract.rs:70-249)
    def packed_tensors(self):
        from ctox_llm_b200.artifact import PackedTensor
        c = self.cfg
        code = {self.orc.Q2B64: "q2_b64", self.orc.Q4B64: "q4_b64"}
        out = []

        def matrix(name, m):
            out.append(PackedTensor(name, code[m.dtype], [m.rows, m.cols], m.packed.tobytes()))
            out.append(PackedTensor(f"{name}.s_in", "f16", [m.cols], np.asarray(m.s_in, np.uint8).tobytes()))
            out.append(PackedTensor(f"{name}.s_out", "f16", [m.rows], np.asarray(m.s_out, np.uint8).tobytes()))

        def vector(name, v, dtype="f32"):
            v = np.asarray(v, np.float32)
            data = v.astype("<f2").tobytes() if dtype == "f16" else v.astype("<f4").tobytes()
            out.append(PackedTensor(name, dtype, [v.size], data))

        matrix("model.language_model.embed_tokens.weight", self.embed)
        matrix("lm_head.weight", self.lm_head)
        vector("model.language_model.norm.weight", self.final_norm)
        for l, L in enumerate(self.layers):
            prefix = "mtp.layers.0" if l >= c.num_hidden_layers else f"model.language_model.layers.{l}"
            vector(f"{prefix}.input_layernorm.weight", L["in_ln"])
            vector(f"{prefix}.post_attention_layernorm.weight", L["post_ln"])
            if L["full"]:
                for p in ("q", "k", "v", "o"):
                    matrix(f"{prefix}.self_attn.{p}_proj.weight", L[p])
                vector(f"{prefix}.self_attn.q_norm.weight", L["q_norm"])
                vector(f"{prefix}.self_attn.k_norm.weight", L["k_norm"])
            else:
                a = f"{prefix}.linear_attn"
                for p, key in (("in_proj_qkv", "qkv"), ("in_proj_z", "z"), ("in_proj_a", "a"), ("in_proj_b", "b"),
                               ("out_proj", "out")):
                    matrix(f"{a}.{p}.weight", L[key])
                vector(f"{a}.conv1d.weight", L["conv_w"])
                vector(f"{a}.A_log", L["a_log"])
                vector(f"{a}.dt_bias", L["dt_bias"])
                vector(f"{a}.norm.weight", L["lin_norm"])
            for p in ("gate", "up", "down"):
                matrix(f"{prefix}.mlp.{p}_proj.weight", L[p])
        if c.mtp_num_hidden_layers:
            matrix("mtp.fc.weight", self.mtp_fc)
            vector("mtp.pre_fc_norm_embedding.weight", self.mtp_norm_e)
            vector("mtp.pre_fc_norm_hidden.weight", self.mtp_norm_h)
            vector("mtp.norm.weight", self.mtp_norm)
        return out

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
                                   "rec": np.zeros(c.linear_num_value_heads * self.kd * self.vd, np.float32)})

    def proj(self, m, x):
        return self.orc.fused_matvec(m.op(self.orc, x), threads=self.threads)

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
        q = np.repeat(conv[: self.kw].reshape(-1, self.kd), rep, axis=0).reshape(-1)
        k = np.repeat(conv[self.kw: 2 * self.kw].reshape(-1, self.kd), rep, axis=0).reshape(-1)
        v = conv[2 * self.kw:]
        g, beta = orc.gated_delta_prepare(a, b, L["a_log"], L["dt_bias"])
        core, st["rec"] = orc.recurrent_gated_delta_step(q, k, v, g, beta, st["rec"], c.linear_num_value_heads,
                                                         self.kd, self.vd)
        core = orc.rms_norm_gated(core, z, c.linear_num_value_heads, self.vd, L["lin_norm"], c.rms_norm_epsilon)
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


    # ---- MTP layer (decoder.rs:1009-1113)
    @staticmethod
    def new_mtp_state():
        """MtpState (decoder.rs:333-337): one full-attention cache that starts one token late."""
        return {"k": [], "v": []}

    def mtp_final_hidden(self, next_token, previous_final_hidden, absolute_position, mst):
        """decoder.rs:1009-1046: fc([norm_e(embed(token)), norm_h(previous hidden)]) -> one
        full-attention layer at rope position `absolute_position`, cache slot = tokens held
        (= absolute_position - 1) -> MLP -> mtp.norm."""
        c = self.cfg
        assert previous_final_hidden.size == c.hidden_size
        assert absolute_position == len(mst["k"]) + 1, "MTP absolute position differs from its cache"
        e = self.norm(self.embedding(int(next_token)), self.mtp_norm_e)
        h = self.norm(np.asarray(previous_final_hidden, np.float32), self.mtp_norm_h)
        x = self.proj(self.mtp_fc, np.concatenate([e, h]))  # embedding first (decoder.rs:1028-1032)
        L = self.layers[c.num_hidden_layers]
        x = self.full_attention(L, x, absolute_position, mst)
        x = self.mlp(L, x)
        return self.norm(x, self.mtp_norm)

    def mtp_draft(self, next_token, previous_final_hidden, absolute_position, mst):
        """decoder.rs:1052-1073: (final hidden, full-vocabulary logits)."""
        fh = self.mtp_final_hidden(next_token, previous_final_hidden, absolute_position, mst)
        return fh, self.proj(self.lm_head, fh)

    def restricted_logits(self, final_hidden, token_ids):
        """decoder.rs:589-627: the lm_head rows of `token_ids` only (same per-row arithmetic)."""
        ids = np.asarray(token_ids, dtype=np.int64)
        assert ids.size and np.all(np.diff(ids) > 0) and ids[-1] < self.cfg.vocab_size
        return self.proj(self.lm_head, final_hidden)[ids]

    def mtp_restricted_draft(self, next_token, previous_final_hidden, absolute_position, mst, token_ids):
        """decoder.rs:1075-1096: (final hidden, logits over the draft vocabulary)."""
        fh = self.mtp_final_hidden(next_token, previous_final_hidden, absolute_position, mst)
        return fh, self.restricted_logits(fh, token_ids)

    def mtp_advance(self, next_token, previous_final_hidden, absolute_position, mst):
        """decoder.rs:1098-1113."""
        self.mtp_final_hidden(next_token, previous_final_hidden, absolute_position, mst)

    def draft_token(self, logits, token_ids=None):
        """DraftDistribution::greedy_token (engine.rs:203-217): the local argmax mapped through the
        strictly increasing id table of a restricted distribution."""
        i = self.orc.greedy_token(np.ascontiguousarray(logits, dtype=np.float32))
        return int(token_ids[i]) if token_ids is not None else int(i)

    def clone_state(self):
        out = []
        for st in self.state:
            if "k" in st:
                out.append({"k": list(st["k"]), "v": list(st["v"])})
            else:
                out.append({"conv": st["conv"].copy(), "rec": st["rec"].copy()})
        return out


def reference_fixture_model(orc, full_layer):
    """The model of the reference's decoder integration test (decoder.rs:1533-1735): constant-valued
    Q2 matrices, zero norm weights, hidden 64, two query heads of 32 over one KV head, one key and
    two value heads of 32 with a 2-tap convolution whose weights are (0, 1), vocabulary of 2, one
    decoder layer (full attention when `full_layer`, else linear attention) and the MTP layer."""
    H = F = 64
    cfg = N.ModelConfig(
        vocab_size=2, hidden_size=H, intermediate_size=F, num_hidden_layers=1, num_attention_heads=2,
        num_key_value_heads=1, head_dim=32, rotary_dim=16, rope_theta=10_000.0, rms_norm_epsilon=1e-6,
        full_attention_interval=1 if full_layer else 4, linear_num_key_heads=1, linear_num_value_heads=2,
        linear_key_head_dim=32, linear_value_head_dim=32, linear_conv_kernel_dim=2,
        mtp_num_hidden_layers=1, max_context_tokens=12, kv_page_tokens=16, kv_dtype=N.F32,
        max_draft_tokens=4, draft_vocab=0)
    m = OracleModel.__new__(OracleModel)
    m.orc, m.cfg, m.kv_bf16, m.threads = orc, cfg, False, 1
    m.qw, m.kvw, m.kd, m.vd = 64, 32, 32, 32
    m.kw, m.vw = 32, 64
    m.channels = 2 * m.kw + m.vw
    Q2 = orc.Q2B64
    K = lambda rows, cols, v: Matrix.constant(orc, Q2, rows, cols, v)
    zeros = lambda n: np.zeros(n, np.float32)
    m.embed = K(2, H, 0.5)
    m.lm_head = K(2, H, 1.0 / H)
    m.final_norm = zeros(H)

    def layer(full, value_scale):
        L = {"full": full, "in_ln": zeros(H), "post_ln": zeros(H),
             "gate": K(F, H, 1.0 / H), "up": K(F, H, value_scale / H), "down": K(H, F, 1.0 / F)}
        if full:
            L.update(q=K(2 * m.qw, H, 1.0 / H), k=K(m.kvw, H, 1.0 / H), v=K(m.kvw, H, value_scale / H),
                     o=K(H, m.qw, 1.0 / m.qw), q_norm=zeros(32), k_norm=zeros(32))
        else:
            L.update(qkv=K(m.channels, H, 1.0 / H), z=K(m.vw, H, 1.0 / H), a=K(2, H, 1.0 / H), b=K(2, H, 1.0 / H),
                     out=K(H, m.vw, 1.0 / m.vw), conv_w=np.tile(np.array([0.0, 1.0], np.float32), m.channels),
                     a_log=zeros(2), dt_bias=zeros(2), lin_norm=np.ones(32, np.float32))
        return L

    # layer 0: up and v weights are 2/hidden; the MTP layer: every projection 1/hidden
    m.layers = [layer(full_layer, 2.0), layer(True, 1.0)]
    m.mtp_fc = K(H, 2 * H, 1.0 / (2 * H))
    m.mtp_norm_e, m.mtp_norm_h, m.mtp_norm = zeros(H), zeros(H), zeros(H)
    m.reset()
    return m


class ReferenceCpuExecutor:
    """CpuCorrectnessExecutor (decoder.rs:1216-1458) on the oracle model: prefill with the MTP cache
    advanced pair by pair, decode with the drafts chained through the TRUE target hidden states
    (decoder.rs:1338-1376), commit by replaying the accepted candidates."""

    def __init__(self, model, draft_tokens, draft_ids=None):
        self.m, self.k = model, draft_tokens
        self.ids = None if draft_ids is None else np.asarray(draft_ids, dtype=np.int64)
        self.mtp = None
        self.last_hidden = None
        self.pending = None

    def prefill(self, tokens, mtp_enabled):  # decoder.rs:1216-1276
        m = self.m
        m.reset()
        self.mtp = m.new_mtp_state() if mtp_enabled else None
        self.last_hidden, self.pending = None, None
        logits = None
        for position, token in enumerate(tokens):
            if mtp_enabled and position > 0:
                m.mtp_advance(token, self.last_hidden, position, self.mtp)
            self.last_hidden, logits = m.decode_target_step(int(token))
        return logits

    def decode(self, token, mtp_enabled):  # decoder.rs:1278-1395
        m = self.m
        assert self.pending is None, "previous speculative branch must be committed"
        draft = None
        if mtp_enabled:
            _, draft = m.mtp_restricted_draft(token, self.last_hidden, m.position, self.mtp, self.ids) \
                if self.ids is not None else m.mtp_draft(token, self.last_hidden, m.position, self.mtp)
        target_hidden, target_logits = m.decode_target_step(int(token))
        out = {"target_logits": target_logits, "draft_logits": [], "target_verification_logits": [],
               "bonus_logits": None, "candidates": []}
        if mtp_enabled:
            saved_state, saved_pos = m.clone_state(), m.position
            mtp_branch = {"k": list(self.mtp["k"]), "v": list(self.mtp["v"])}
            cur_hidden, cur_logits = target_hidden, target_logits
            for depth in range(self.k):
                out["target_verification_logits"].append(cur_logits)
                candidate = m.draft_token(draft, self.ids)
                out["draft_logits"].append(draft)
                out["candidates"].append(candidate)
                if depth + 1 < self.k:
                    if self.ids is not None:
                        _, draft = m.mtp_restricted_draft(candidate, cur_hidden, m.position, mtp_branch, self.ids)
                    else:
                        _, draft = m.mtp_draft(candidate, cur_hidden, m.position, mtp_branch)
                cur_hidden, cur_logits = m.decode_target_step(candidate)
            out["bonus_logits"] = cur_logits
            m.state, m.position = saved_state, saved_pos  # the branch is dropped
            self.pending = list(out["candidates"])
        self.last_hidden = target_hidden
        return out

    def commit_speculative(self, accepted):  # decoder.rs:1397-1458
        assert self.pending is not None, "no pending speculative branch"
        cands, self.pending = self.pending, None
        assert accepted <= len(cands)
        for candidate in cands[:accepted]:
            self.m.mtp_advance(candidate, self.last_hidden, self.m.position, self.mtp)
            self.last_hidden, _ = self.m.decode_target_step(candidate)


class DeviceChainOracle:
    """The speculative block as an accelerator runs it, on the oracle model: the first draft from
    the pair (token, last target hidden) like the CPU executor; drafts 2..k chained through the
    MTP layer's OWN final hidden (backend/cuda_graph.rs:4258-4262), on a branch of the MTP cache;
    one verify pass; greedy acceptance (engine.rs:939-962); the accepted prefix committed, and the
    MTP cache advanced over the committed pairs with the target's true hidden states at the start
    of the next block (which leaves the cache as decoder.rs:1216-1276,1397-1458 leave it)."""

    def __init__(self, model, draft_tokens, draft_ids=None):
        self.m, self.k = model, draft_tokens
        self.ids = None if draft_ids is None else np.asarray(draft_ids, dtype=np.int64)

    def prefill(self, tokens, chunk=8):
        """The last token is the first decode's input. The target runs in chunks of `chunk`
        positions; the MTP cache is advanced after every chunk but the last, whose pairs are owed
        to the first decode's catch-up pass (the cache ends up the same either way)."""
        m = self.m
        m.reset()
        self.mtp = m.new_mtp_state()
        consume = len(tokens) - 1
        last_chunk_start = (consume - 1) // chunk * chunk if consume else 0
        hiddens = []
        for position in range(consume):
            hidden, _ = m.decode_target_step(int(tokens[position]))
            hiddens.append(hidden)
        # pair of absolute position p: (token p, final hidden of position p - 1)
        for p in range(1, last_chunk_start + 1):
            m.mtp_advance(tokens[p], hiddens[p - 1], p, self.mtp)
        self.owed = [(int(tokens[p]), hiddens[p - 1]) for p in range(last_chunk_start + 1, consume)]
        self.last_hidden = hiddens[-1] if hiddens else None

    def _logits(self, fh):
        return self.m.restricted_logits(fh, self.ids) if self.ids is not None else self.m.proj(self.m.lm_head, fh)

    def decode(self, token, force_accept=-1, given_drafts=None):
        """Returns a dict with the MTP hidden of every pair in the order the device runs them, the
        draft logits and tokens, the target's greedy token per verify position, the accepted count
        and the emitted tokens. given_drafts: follow these draft tokens instead of the oracle's own
        (teacher forcing, when a near-tie made the device pick another token)."""
        m, P = self.m, self.m.position
        mtp_hidden, draft_logits, drafts = [], [], []
        pairs = self.owed + [(int(token), self.last_hidden)]
        fh = None
        for j, (tok, hid) in enumerate(pairs):
            fh = m.mtp_final_hidden(tok, hid, P - len(pairs) + 1 + j, self.mtp)
            mtp_hidden.append(fh)
        branch = {"k": list(self.mtp["k"]), "v": list(self.mtp["v"])}
        for i in range(self.k):
            lg = self._logits(fh)
            draft_logits.append(lg)
            own = m.draft_token(lg, self.ids)
            drafts.append(own)
            follow = own if given_drafts is None else int(given_drafts[i])
            if i + 1 < self.k:
                fh = m.mtp_final_hidden(follow, fh, P + 1 + i, branch)
                mtp_hidden.append(fh)
        followed = drafts if given_drafts is None else [int(d) for d in given_drafts]
        # verify: the target over [token, drafts...] while the prefix is accepted
        hiddens, target_tokens, accepted, target_logits = [], [], [], []
        hidden, logits = m.decode_target_step(int(token))
        hiddens.append(hidden)
        target_logits.append(logits)
        target_tokens.append(m.orc.greedy_token(logits))
        for i in range(self.k):
            ok = followed[i] == target_tokens[-1] if force_accept < 0 else i < force_accept
            if not ok:
                break
            accepted.append(followed[i])
            hidden, logits = m.decode_target_step(followed[i])
            hiddens.append(hidden)
            target_logits.append(logits)
            target_tokens.append(m.orc.greedy_token(logits))
        next_token = target_tokens[-1]
        self.owed = [(accepted[j], hiddens[j]) for j in range(len(accepted))]
        self.last_hidden = hiddens[-1]
        return {"mtp_hidden": mtp_hidden, "draft_logits": draft_logits, "drafts": drafts,
                "target_tokens": target_tokens, "accepted": accepted, "next_token": next_token,
                "final_hidden": hiddens[-1], "target_logits": target_logits}
