"""Model families on CPU: every registered family builds from its preset, trains a few steps
through the ZeRO engine, and the family-specific pieces (sinks / sliding window attention,
group-limited sigmoid routing with a selection bias, clamped SwiGLU with expert biases, MLA)
match independent PyTorch restatements."""
import math
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


@pytest.fixture(autouse=True)
def _state():
    from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state
    reset_parallel_state()
    init_parallel_state(device_type="cpu")
    yield
    reset_parallel_state()


@pytest.mark.parametrize("name", ["tiny-qwen3", "tiny-qwen2", "tiny-olmo2", "tiny-qwen3-moe", "tiny-gpt-oss",
                                  "tiny-deepseek-v3", "tiny-glm4-moe", "tiny-qwen3-5", "tiny-qwen3-5-moe",
                                  "tiny-nemotron-h", "tiny-minimax-m3", "tiny-glm5", "tiny-deepseek-v4"])
def test_family_trains(name):
    from xorl_b200.models import build_model
    from xorl_b200.models.config import preset
    from xorl_b200.optim import build_optimizer
    from xorl_b200.parallel.state import get_parallel_state
    from xorl_b200.parallel.zero import Zero3Engine
    cfg = preset(name)
    from xorl_b200.models.registry import get_model_class
    m = get_model_class(cfg)(cfg, dtype=torch.float32, device="meta")
    eng = Zero3Engine(m, get_parallel_state(), compute_dtype=torch.float32, device=torch.device("cpu"), seed=0)
    opt = build_optimizer(eng, lr=3e-3, weight_decay=0.0)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (1, 49), generator=g)
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    cu = torch.tensor([0, 20, 48], dtype=torch.int32)
    pos = torch.cat([torch.arange(20), torch.arange(28)]).unsqueeze(0)
    losses = []
    for _ in range(5):
        opt.zero_grad()
        loss = eng.forward_backward(x, y, position_ids=pos, cu_seqlens=cu, grad_scale=1.0 / y.numel())
        eng.finish_grad_sync()
        opt.step()
        losses.append(float(loss))
    assert all(math.isfinite(l) for l in losses) and losses[-1] < losses[0], losses


def test_unknown_family_fails_loudly():
    from xorl_b200.models.config import ModelConfig
    from xorl_b200.models.registry import get_model_class
    with pytest.raises(KeyError):
        get_model_class(ModelConfig.from_dict({"model_type": "not_a_model"}))


def test_deepseek_v4_pieces():
    """Hyper-connection mixers (Sinkhorn-normalised mixing matrix, collapse / spread algebra), the
    pooled key compressor against its definition, the window-only attention layer against dense
    attention with a window and sink logits on a shared key/value head, and hash routing."""
    from xorl_b200.models import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.models.deepseek_v4 import HyperConnection, hc_split_sinkhorn, rope_tables, rope_tail
    from xorl_b200.ops.attention import attention_reference
    torch.manual_seed(0)
    hc = 4
    mixes = torch.randn(7, (2 + hc) * hc)
    pre, post, comb = hc_split_sinkhorn(mixes, torch.tensor([1.0, 0.5, 2.0]), torch.randn((2 + hc) * hc) * 0.1, hc, 20, 1e-6)
    assert pre.shape == (7, hc) and (pre > 0).all() and (post > 0).all() and (post < 2).all()
    assert (comb.sum(-1) - 1).abs().max() < 5e-3 and (comb.sum(-2) - 1).abs().max() < 1e-4   # columns were normalised last
    x, y = torch.randn(7, hc, 5), torch.randn(7, 5)
    out = HyperConnection.post(y, x, post, comb)
    ref = torch.stack([post[:, i:i + 1] * y + sum(comb[:, j, i:i + 1] * x[:, j] for j in range(hc)) for i in range(hc)], 1)
    assert (out - ref).abs().max() < 1e-5
    # rotating the tail and rotating back is the identity
    t = torch.randn(6, 2, 16)
    cos, sin = rope_tables(torch.arange(6), 8, 1e4)
    assert (rope_tail(rope_tail(t, cos, sin, 8), cos, sin, 8, inverse=True) - t).abs().max() < 1e-5
    cfg = preset("tiny-deepseek-v4")
    m = DecoderLM(cfg)
    m.init_weights(0)
    ids = torch.randint(0, cfg.vocab_size, (40,))
    cu = torch.tensor([0, 40], dtype=torch.int32)
    ctx = m.make_context(ids, cu_seqlens=cu)
    # compressor of layer 2 would need 128 tokens; layer 1 (ratio 4, overlapping groups)
    comp = m.layers["1"].self_attn.compressor
    xin = torch.randn(40, cfg.hidden_size)
    got = comp(xin, ctx.position_ids)
    assert got.shape == (10, cfg.extra["v4_head_dim"])
    hd = comp.hd
    kv = torch.nn.functional.linear(xin, comp.wkv.weight).view(10, 4, 2 * hd)
    sc = torch.nn.functional.linear(xin, comp.wgate.weight).view(10, 4, 2 * hd) + comp.ape
    g = 3                                                   # group 3 pools its own 4 tokens and group 2's
    slots_kv = torch.cat([kv[g - 1, :, :hd], kv[g, :, hd:]], 0)
    slots_sc = torch.cat([sc[g - 1, :, :hd], sc[g, :, hd:]], 0)
    pooled = comp.norm((slots_kv * slots_sc.softmax(0)).sum(0, keepdim=True))
    c4, s4 = rope_tables(torch.tensor([g * 4]), comp.rd, comp.theta)
    assert (rope_tail(pooled.unsqueeze(1), c4, s4, comp.rd)[0, 0] - got[g]).abs().max() < 1e-5
    # layer 0: sliding window + sinks only
    att = m.layers["0"].self_attn
    with torch.no_grad():
        att.attn_sink.copy_(torch.randn(att.H))
        h = torch.randn(40, cfg.hidden_size)
        out = att(h, ctx)
        cos, sin = rope_tables(ctx.position_ids, att.rd, att.theta)
        q = att.wq_b(att.q_norm(att.wq_a(h))).view(40, att.H, att.hd)
        q = rope_tail(q * torch.rsqrt(q.square().mean(-1, keepdim=True) + att.eps), cos, sin, att.rd)
        kv1 = rope_tail(att.kv_norm(att.wkv(h)).unsqueeze(1), cos, sin, att.rd)
        o = attention_reference(q, kv1, kv1, cu, True, att.scale, window=att.window, sinks=att.attn_sink)
        o = rope_tail(o, cos, sin, att.rd, inverse=True).reshape(40, att.G, -1)
        ref = att.wo_b(torch.einsum("tgd,grd->tgr", o, att.wo_a.weight.view(att.G, att.r_o, -1)).reshape(40, -1))
    assert (out - ref).abs().max() < 1e-4
    # hash routing: layer 0 sends every token to the experts listed for its id
    moe = m.layers["0"].mlp
    assert moe.is_hash_layer and not m.layers["1"].mlp.is_hash_layer
    ctx.aux["collect_expert_load"] = True
    with torch.no_grad():
        moe(torch.randn(40, cfg.hidden_size), ctx)
    want = torch.bincount(moe.tid2eid[ids].long().reshape(-1), minlength=cfg.num_experts)
    assert torch.equal(ctx.aux[("expert_load", 0)], want)


def test_attention_window_and_sinks_reference():
    from xorl_b200.ops.attention import attention_reference
    torch.manual_seed(0)
    T, Hq, Hkv, D = 12, 4, 2, 8
    q, k, v = torch.randn(T, Hq, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    sinks = torch.randn(Hq)
    cu = torch.tensor([0, 5, 12], dtype=torch.int32)
    out = attention_reference(q, k, v, cu, True, 0.3, window=3, sinks=sinks)
    # token by token
    for (s, e) in ((0, 5), (5, 12)):
        for t in range(s, e):
            lo = max(s, t - 2)
            for h in range(Hq):
                kk, vv = k[lo:t + 1, h // 2], v[lo:t + 1, h // 2]
                logits = torch.cat([(kk @ q[t, h]) * 0.3, sinks[h:h + 1]])
                p = torch.softmax(logits, 0)[:-1]
                torch.testing.assert_close(out[t, h], p @ vv, rtol=1e-5, atol=1e-5)


def test_group_limited_sigmoid_routing():
    from xorl_b200.ops.moe import topk_route
    torch.manual_seed(1)
    T, E, k = 16, 8, 2
    logits = torch.randn(T, E)
    bias = torch.randn(E) * 0.5
    w, idx, probs = topk_route(logits, k, True, "sigmoid", 2.5, n_group=4, topk_group=2, correction_bias=bias)
    s = torch.sigmoid(logits)
    for t in range(T):
        c = s[t] + bias
        gs = c.view(4, 2).sum(-1)                              # two experts per group: top-2 sum = sum
        groups = set(gs.topk(2)[1].tolist())
        allowed = [e for e in range(E) if e // 2 in groups]
        best = sorted(allowed, key=lambda e: -c[e].item())[:k]
        assert set(idx[t].tolist()) == set(best)
        ww = s[t, idx[t]]
        torch.testing.assert_close(w[t], ww / ww.sum() * 2.5)
    # gpt-oss style: softmax over the selected logits only
    w2, idx2, _ = topk_route(logits, k, False, "softmax_after_topk")
    torch.testing.assert_close(w2, torch.softmax(logits.topk(k)[0], -1))


def test_clamped_swiglu_expert_mlp_with_biases():
    from xorl_b200.ops import moe as moe_ops
    torch.manual_seed(2)
    E, H, I = 3, 16, 8
    counts = torch.tensor([5, 0, 7])
    x = torch.randn(12, H)
    gu, dn = torch.randn(E, H, 2 * I) * 0.3, torch.randn(E, I, H) * 0.3
    gub, dnb = torch.randn(E, 2 * I), torch.randn(E, H)
    y = moe_ops.expert_mlp(x, counts, gu, dn, gate_up_bias=gub, down_bias=dnb, swiglu_limit=1.5)
    s = 0
    for e in range(E):
        n = counts[e].item()
        xe = x[s:s + n]
        h = xe @ gu[e] + gub[e]
        gate, up = h[:, :I].clamp(max=1.5), h[:, I:].clamp(-1.5, 1.5)
        ref = ((up + 1) * gate * torch.sigmoid(1.702 * gate)) @ dn[e] + dnb[e]
        torch.testing.assert_close(y[s:s + n], ref, rtol=1e-4, atol=1e-4)
        s += n


def test_mla_matches_explicit_formula():
    from xorl_b200.models.config import preset
    from xorl_b200.models.context import StepContext
    from xorl_b200.models.mla import MLAttention
    from xorl_b200.models.rope import RotaryEmbedding
    cfg = preset("tiny-deepseek-v3")
    torch.manual_seed(3)
    m = MLAttention(cfg, 0, dtype=torch.float32)
    for p in m.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.2)
    T = 6
    x = torch.randn(T, cfg.hidden_size)
    rot = RotaryEmbedding(cfg.head_dim, cfg.rope_theta, None, 1.0, 512)
    cos, sin = rot(torch.arange(T))
    ctx = StepContext(cu_seqlens=torch.tensor([0, T], dtype=torch.int32), position_ids=torch.arange(T),
                      max_seqlen=T, cos=cos, sin=sin)
    out = m(x, ctx)
    # explicit: complex rotation on interleaved pairs, per-head loop
    H, dn, dr, dv = 4, 16, 8, 16
    q = m.q_b_proj(m.q_a_layernorm(m.q_a_proj(x))).view(T, H, dn + dr)
    ckv = m.kv_a_proj_with_mqa(x)
    c, kr = ckv[:, :24], ckv[:, 24:]
    kv = m.kv_b_proj(m.kv_a_layernorm(c)).view(T, H, dn + dv)
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, dr, 2).float() / dr))
    ang = torch.arange(T).float()[:, None] * inv[None]
    rotc = torch.polar(torch.ones_like(ang), ang)                        # [T, dr/2]

    def rope_interleaved(t):                                              # [T, h, dr]
        z = torch.view_as_complex(t.reshape(*t.shape[:-1], dr // 2, 2).contiguous())
        return z * rotc[:, None, :]

    qr = rope_interleaved(q[..., dn:])
    krr = rope_interleaved(kr.reshape(T, 1, dr))
    ref = torch.zeros(T, H, dv)
    for h in range(H):
        s_nope = q[:, h, :dn] @ kv[:, h, :dn].t()
        s_rope = torch.einsum("ic,jc->ij", qr[:, h], krr[:, 0].conj()).real
        sc = (s_nope + s_rope) * (dn + dr) ** -0.5
        sc = sc.masked_fill(~torch.ones(T, T, dtype=torch.bool).tril(), float("-inf"))
        ref[:, h] = torch.softmax(sc, -1) @ kv[:, h, dn:]
    ref = m.o_proj(ref.reshape(T, H * dv))
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("name", ["tiny-gpt-oss", "tiny-deepseek-v3", "tiny-qwen3-moe", "tiny-qwen3-5", "tiny-qwen3-5-moe", "tiny-nemotron-h",
                                  "tiny-minimax-m3", "tiny-glm5", "tiny-deepseek-v4"])
def test_family_hf_roundtrip(name, tmp_path):
    """Export to HF-named safetensors and load back into a fresh engine: identical weights."""
    from xorl_b200.checkpoint.hf_io import load_hf_weights, save_hf_weights
    from xorl_b200.models.config import preset
    from xorl_b200.models.registry import get_model_class
    from xorl_b200.parallel.state import get_parallel_state
    from xorl_b200.parallel.zero import Zero3Engine
    cfg = preset(name)

    def engine(seed):
        m = get_model_class(cfg)(cfg, dtype=torch.float32, device="meta")
        return Zero3Engine(m, get_parallel_state(), compute_dtype=torch.float32, device=torch.device("cpu"), seed=seed)

    a, b = engine(0), engine(1)
    save_hf_weights(a, str(tmp_path), cfg, dtype=torch.float32)
    from safetensors import safe_open
    names = []
    for f in os.listdir(tmp_path):
        if f.endswith(".safetensors"):
            with safe_open(str(tmp_path / f), "pt") as fh:
                names += list(fh.keys())
    if name == "tiny-gpt-oss":
        assert "model.layers.0.mlp.router.weight" in names and "model.layers.0.mlp.experts.gate_up_proj_bias" in names
        assert "model.layers.0.self_attn.sinks" in names
    if name.startswith("tiny-qwen3-5"):
        assert "model.layers.0.linear_attn.in_proj_qkv.weight" in names and "model.layers.0.linear_attn.conv1d.weight" in names
        assert "model.layers.0.linear_attn.in_proj_z.weight" in names and "model.layers.0.linear_attn.A_log" in names
        assert "model.layers.3.self_attn.q_proj.weight" in names and not any("out_gate" in n or "qkv_proj" in n for n in names)
    if name == "tiny-deepseek-v4":
        for n in ("model.layers.0.hc_attn_fn", "model.layers.3.hc_ffn_scale", "model.hc_head_base",
                  "model.layers.0.mlp.tid2eid", "model.layers.1.mlp.gate.e_score_correction_bias",
                  "model.layers.1.self_attn.indexer.compressor.ape", "model.layers.2.self_attn.compressor.wgate.weight",
                  "model.layers.0.self_attn.attn_sink", "model.layers.1.mlp.shared_experts.down_proj.weight"):
            assert n in names, n
    if name == "tiny-glm5":
        for n in ("model.layers.0.self_attn.indexer.k_norm.bias", "model.layers.0.self_attn.indexer.wq_b.weight",
                  "model.layers.2.self_attn.indexer.weights_proj.weight", "model.layers.1.mlp.shared_experts.up_proj.weight",
                  "model.layers.1.self_attn.kv_a_proj_with_mqa.weight"):
            assert n in names, n
        assert not any(n.startswith("model.layers.1.self_attn.indexer") for n in names)     # shares layer 0's selection
    if name == "tiny-minimax-m3":
        for n in ("model.layers.0.mlp.gate_proj.weight", "model.layers.1.block_sparse_moe.experts.3.w1.weight",
                  "model.layers.1.block_sparse_moe.experts.3.w2.weight", "model.layers.1.block_sparse_moe.gate.weight",
                  "model.layers.1.block_sparse_moe.e_score_correction_bias",
                  "model.layers.1.block_sparse_moe.shared_experts.up_proj.weight",
                  "model.layers.1.self_attn.index_q_proj.weight", "model.layers.1.self_attn.q_norm.weight"):
            assert n in names, n
    if name == "tiny-nemotron-h":
        for n in ("backbone.embeddings.weight", "backbone.norm_f.weight", "backbone.layers.0.mixer.conv1d.weight",
                  "backbone.layers.0.mixer.A_log", "backbone.layers.0.mixer.norm.weight",
                  "backbone.layers.1.mixer.experts.5.up_proj.weight", "backbone.layers.1.mixer.fc1_latent_proj.weight",
                  "backbone.layers.1.mixer.shared_experts.down_proj.weight", "backbone.layers.1.mixer.gate.e_score_correction_bias",
                  "backbone.layers.2.mixer.k_proj.weight", "backbone.layers.3.mixer.up_proj.weight", "lm_head.weight"):
            assert n in names, n
    if name == "tiny-deepseek-v3":
        assert "model.layers.1.mlp.shared_experts.gate_proj.weight" in names
        assert "model.layers.1.mlp.experts.3.down_proj.weight" in names
        assert "model.layers.1.mlp.gate.e_score_correction_bias" in names
    missing = load_hf_weights(b, str(tmp_path), cfg)
    assert not missing
    wa = dict(a.iter_full_tensors("master"))
    for k, v in b.iter_full_tensors("master"):
        assert torch.equal(v, wa[k]), k


def test_glm5_indexer_selection_and_sharing():
    """The lightning indexer keeps the top-k causal keys of every query, by the gated ReLU score;
    layers without an indexer attend to the selection of the closest earlier layer that has one;
    with top-k >= document length the model equals dense latent attention."""
    from xorl_b200.models import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.models.glm5 import indexer_scores, select_topk_keys
    torch.manual_seed(0)
    L, Hi, Di = 20, 2, 8
    iq, ik, g = torch.randn(L, Hi, Di), torch.randn(L, Di), torch.rand(L, Hi)
    sc = indexer_scores(iq, ik, g)
    ref = torch.zeros(L, L)
    for t in range(L):
        for s_ in range(L):
            ref[t, s_] = sum(g[t, h] * torch.relu(iq[t, h] @ ik[s_]) for h in range(Hi)) * Di ** -0.5
    assert (sc - ref).abs().max() < 1e-5
    keep = select_topk_keys(sc, 4)
    assert keep.sum(-1).tolist() == [min(t + 1, 4) for t in range(L)] and not keep.triu(1).any()
    t = 15
    best = sc[t, : t + 1].topk(4).indices.sort().values
    assert torch.equal(keep[t].nonzero().flatten(), best)
    cfg = preset("tiny-glm5")
    m = DecoderLM(cfg)
    m.init_weights(0)
    ids = torch.randint(0, cfg.vocab_size, (48,))
    cu = torch.tensor([0, 20, 48], dtype=torch.int32)
    with torch.no_grad():
        sparse = m.logits(ids, cu_seqlens=cu)
        for l in m.layers.values():
            if l.self_attn.indexer is not None:
                l.self_attn.indexer.topk = 1000
        dense = m.logits(ids, cu_seqlens=cu)
        ctx = m.make_context(ids, cu_seqlens=cu)
        h, r = m.forward_embed(ids, ctx)
        for l in m.layers.values():
            h, r = l(h, r, ctx)
    assert (sparse[:8] - dense[:8]).abs().max() < 1e-4         # the first 8 tokens see at most 8 keys
    assert (sparse - dense).abs().max() > 1e-4
    assert ("dsa_keep", 0) in ctx.aux and ("dsa_keep", 2) in ctx.aux and ("dsa_keep", 1) not in ctx.aux
    assert m.layers["1"].self_attn.indexer is None and m.layers["1"].self_attn.producer == 0


def test_minimax_sparse_attention_selects_blocks():
    """Block-sparse inference attention: with enough blocks kept it equals dense causal attention;
    with few it attends only inside the kept blocks (forced first block, own block, best-scoring)."""
    from xorl_b200.models.minimax_m3 import msa_attention
    from xorl_b200.ops.attention import attention_reference
    torch.manual_seed(0)
    T, Hq, Hkv, D, Hi, Di, bs = 70, 4, 2, 8, 2, 8, 8
    q, k, v = torch.randn(T, Hq, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    iq, ik = torch.randn(T, Hi, Di), torch.randn(T, Hi, Di)
    cu = torch.tensor([0, 30, 70], dtype=torch.int32)
    dense = attention_reference(q, k, v, cu, True, D ** -0.5)
    full = msa_attention(q, k, v, iq, ik, cu, D ** -0.5, block_size=bs, topk_blocks=16)
    assert (full - dense).abs().max() < 1e-5
    # one kept block = the query's own block (forced): equals attention restricted to that block
    own = msa_attention(q, k, v, iq, ik, cu, D ** -0.5, block_size=bs, topk_blocks=1, force_end_blocks=1)
    t = 29                       # last token of the first document: block 3 = keys 24..29
    kh = k[24:30].repeat_interleave(2, 1)
    vh = v[24:30].repeat_interleave(2, 1)
    att = (torch.einsum("hd,khd->hk", q[t], kh) * D ** -0.5).softmax(-1)
    assert (own[t] - torch.einsum("hk,khd->hd", att, vh)).abs().max() < 1e-5
    sparse = msa_attention(q, k, v, iq, ik, cu, D ** -0.5, block_size=bs, topk_blocks=2, force_begin_blocks=1)
    assert torch.isfinite(sparse).all() and (sparse - dense).abs().max() > 1e-3


def test_minimax_model_sparse_inference_path():
    from xorl_b200.models import preset
    from xorl_b200.models.decoder import DecoderLM
    torch.manual_seed(0)
    cfg = preset("tiny-minimax-m3")
    m = DecoderLM(cfg)
    m.init_weights(0)
    assert m.layers["1"].self_attn.is_sparse_layer and not m.layers["0"].self_attn.is_sparse_layer
    assert m.layers["1"].self_attn.q_norm.weight.shape == (cfg.num_attention_heads * cfg.head_dim,)
    ids = torch.randint(0, cfg.vocab_size, (64,))
    cu = torch.tensor([0, 64], dtype=torch.int32)
    with torch.no_grad():
        dense = m.logits(ids, cu_seqlens=cu)
        m.ctx_defaults["minimax_msa"] = True
        sparse = m.logits(ids, cu_seqlens=cu)
    assert torch.isfinite(sparse).all() and (sparse - dense).abs().max() > 1e-6
    assert (sparse[:16] - dense[:16]).abs().max() < 1e-4      # two blocks of 8 are always kept: same as dense


def test_mamba2_chunked_scan_matches_recurrence():
    """Chunked state-space scan (several chunk sizes, documents shorter and longer than a chunk,
    a one-token document) against the token-by-token recurrence, values and gradients."""
    from xorl_b200.models.mamba2 import segment_ids, ssd_chunked, ssd_reference
    torch.manual_seed(0)
    T, H, P, G, N = 150, 4, 8, 2, 6
    x = torch.randn(T, H, P, requires_grad=True)
    dt = (torch.rand(T, H) * 0.5 + 0.01).requires_grad_(True)
    A = -torch.rand(H) * 2 - 0.1
    B, C, D = torch.randn(T, G, N), torch.randn(T, G, N), torch.randn(H)
    seg = segment_ids(torch.tensor([0, 37, 64, 65, 140]), T)
    ref = ssd_reference(x, dt, A, B, C, D, seg)
    gx, gdt = torch.autograd.grad(ref.square().sum(), (x, dt))
    for q in (16, 32, 64):
        got = ssd_chunked(x, dt, A, B, C, D, seg, q)
        assert (got - ref).abs().max() < 1e-4
        hx, hdt = torch.autograd.grad(got.square().sum(), (x, dt))
        assert (hx - gx).abs().max() < 1e-3 and (hdt - gdt).abs().max() < 5e-3
        assert torch.isfinite(hdt).all()


def test_nemotron_h_trains_and_keeps_documents_apart():
    """Mamba2 / attention without rotary embedding / latent relu^2 MoE / MLP blocks: the loss falls on
    a fixed batch, and a document's logits do not depend on the document packed before it."""
    from xorl_b200.models import preset
    from xorl_b200.models.decoder import DecoderLM
    torch.manual_seed(0)
    cfg = preset("tiny-nemotron-h")
    assert cfg.num_hidden_layers == 6 and cfg.layer_is_moe(1) and not cfg.layer_is_moe(0)
    m = DecoderLM(cfg)
    m.init_weights(0)
    ids = torch.randint(0, cfg.vocab_size, (96,))
    cu = torch.tensor([0, 40, 96], dtype=torch.int32)
    with torch.no_grad():
        full = m.logits(ids, cu_seqlens=cu)
        alone = m.logits(ids[40:], cu_seqlens=torch.tensor([0, 56], dtype=torch.int32))
    assert (full[40:] - alone).abs().max() < 1e-4
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    losses = []
    for _ in range(8):
        opt.zero_grad()
        out = m(ids[:-1], labels=ids[1:], cu_seqlens=torch.tensor([0, 40, 95], dtype=torch.int32), grad_scale=1 / 95)
        out["loss"].backward()
        opt.step()
        losses.append(float(out["loss"].detach()))
    assert losses[-1] < losses[0] - 0.3, losses


def test_gated_delta_rule_matches_dense_formula():
    """The recurrence against an explicit per-head float64 restatement, with a document boundary."""
    from xorl_b200.models.gated_deltanet import causal_depthwise_conv, gated_delta_rule
    torch.manual_seed(0)
    T, H, dk, dv = 11, 3, 4, 5
    q, k = torch.randn(T, H, dk), torch.nn.functional.normalize(torch.randn(T, H, dk), dim=-1)
    v, g, beta = torch.randn(T, H, dv), -torch.rand(T, H), torch.rand(T, H)
    cu = torch.tensor([0, 4, 11], dtype=torch.int32)
    out = gated_delta_rule(q, k, v, g, beta, cu)
    for h in range(H):
        for (s, e) in ((0, 4), (4, 11)):
            S = torch.zeros(dk, dv, dtype=torch.float64)
            for t in range(s, e):
                S = math.exp(g[t, h].item()) * S
                kt = k[t, h].double()
                S = S + torch.outer(kt, beta[t, h].double() * (v[t, h].double() - S.t() @ kt))
                torch.testing.assert_close(out[t, h].double(), S.t() @ q[t, h].double(), rtol=1e-5, atol=1e-5)
    # the convolution is causal and does not cross documents
    x = torch.randn(T, 6)
    w = torch.randn(6, 4)
    y = causal_depthwise_conv(x, w, cu)
    t = 5                                                     # second token of the second document
    ref = w[:, 3] * x[5] + w[:, 2] * x[4]
    torch.testing.assert_close(y[t], ref)


@pytest.mark.parametrize("chunk", [8, 64])
def test_chunked_gated_delta_rule_matches_recurrence(chunk):
    """The chunked form against the token recurrence: outputs, every gradient, and the state handed
    from one half of a document to the other."""
    from xorl_b200.models.gated_deltanet import gated_delta_rule, gated_delta_rule_chunked
    torch.manual_seed(1)
    T, H, dk, dv = 150, 2, 8, 12
    cu = torch.tensor([0, 37, 38, 130, 141], dtype=torch.int32)      # the last 9 tokens are padding
    mk = lambda *s: torch.randn(*s, dtype=torch.float64)
    q = torch.nn.functional.normalize(mk(T, H, dk), dim=-1).requires_grad_()
    k = torch.nn.functional.normalize(mk(T, H, dk), dim=-1).requires_grad_()
    v = mk(T, H, dv).requires_grad_()
    g = (-torch.rand(T, H, dtype=torch.float64)).requires_grad_()
    beta = torch.rand(T, H, dtype=torch.float64).requires_grad_()
    ref = gated_delta_rule(q, k, v, g, beta, cu)
    out = gated_delta_rule_chunked(q, k, v, g, beta, cu, chunk=chunk)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)
    w = mk(T, H, dv)
    g_ref = torch.autograd.grad((ref * w).sum(), [q, k, v, g, beta])
    g_out = torch.autograd.grad((out * w).sum(), [q, k, v, g, beta])
    for a, b in zip(g_out, g_ref):
        torch.testing.assert_close(a, b, rtol=1e-3, atol=1e-4)
    # one document of 92 tokens cut at token 50: the second half started from the first half's state
    sl = lambda x, a, b: x[a:b].detach()
    one = torch.tensor([0, 92], dtype=torch.int32)
    full = gated_delta_rule_chunked(*(sl(x, 38, 130) for x in (q, k, v, g, beta)), one, chunk=chunk)
    h1, S = gated_delta_rule_chunked(*(sl(x, 38, 88) for x in (q, k, v, g, beta)),
                                     torch.tensor([0, 50]), chunk=chunk, return_final_state=True)
    h2 = gated_delta_rule_chunked(*(sl(x, 88, 130) for x in (q, k, v, g, beta)),
                                  torch.tensor([0, 42]), chunk=chunk, initial_state=S)
    torch.testing.assert_close(torch.cat([h1, h2]), full, rtol=1e-4, atol=1e-5)


def test_causal_conv1d_tensor_form_matches_per_document_convolution():
    from xorl_b200.models.gated_deltanet import causal_depthwise_conv
    from xorl_b200.ops.seqmix import causal_conv1d, document_starts
    torch.manual_seed(2)
    T, C, K = 40, 16, 4
    cu = torch.tensor([0, 1, 14, 33], dtype=torch.int32)
    assert document_starts(cu, T).tolist() == [0] + [1] * 13 + [14] * 19 + list(range(33, 40))
    x, w, b = torch.randn(T, C), torch.randn(C, K), torch.randn(C)
    y = causal_conv1d(x, w, b, cu, silu=True)
    ref = torch.nn.functional.silu(causal_depthwise_conv(x, w, cu) + b)
    torch.testing.assert_close(y[:33], ref[:33], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(y[35], torch.nn.functional.silu(w[:, 3] * x[35] + b), rtol=1e-5, atol=1e-5)
