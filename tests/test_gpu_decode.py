"""Whole-token decode path (mb200_decode_*): every layer against the oracle's restatement of the
reference's op order (src/forward.c:670-823, 1114), the sampled tokens against a greedy decode by
the oracle, and CUDA-graph replay against eager execution. Model tensors are written on the
device by the library's fill kernels and copied to the host for the oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from mnemocuda_b200 import kernels
    kernels.mb200_init()
    yield kernels
    torch.cuda.synchronize()
    assert kernels.mb200_device_error() == 0


def host_layer(model, l):
    T = model.layers[l]
    L = {k: T[k].cpu().numpy() for k in ("attn_norm", "wq", "wk", "wv", "wo", "q_norm", "k_norm", "ffn_norm")}
    L["router"] = T["router"].reshape(-1).cpu().numpy()
    L["experts"] = T["experts"].reshape(-1).cpu().numpy()
    return L


def cfg_dict(c):
    g, u, d = c.expert_sizes()
    return dict(hidden=c.hidden, n_heads=c.n_heads, n_kv_heads=c.n_kv_heads, head_dim=c.head_dim, rms_eps=c.rms_eps,
                rope_theta=c.rope_theta, wq_type=c.wq_type, wk_type=c.wk_type, wv_type=c.wv_type, wo_type=c.wo_type,
                expert_stride=c.expert_stride, gate_sz=g, up_sz=u, down_type=c.down_type, n_experts=c.n_experts,
                top_k=c.top_k, moe_inter=c.moe_inter)


def oracle_token(model, Ls, kv, token, pos):
    """One greedy token by the oracle; kv: per-layer (k_bits, v_bits) host caches, updated in place."""
    c = model.cfg
    h = oracle.embedding_q4k(model.token_embd.cpu().numpy(), token, c.hidden)
    for l in range(c.n_layers):
        h, _ = oracle.decode_layer(h, Ls[l], cfg_dict(c), pos, kv[l][0], kv[l][1])
    normed = oracle.rms_norm(h, model.output_norm.cpu().numpy(), c.rms_eps)
    mv = oracle.matvec_q6k if c.lm_head_type == 14 else oracle.matvec_q4k
    logits = mv(model.lm_head.cpu().numpy(), normed, c.vocab, c.hidden)
    return oracle.argmax(logits), logits, h


SHAPES = {
    # fused MoE kernel not applicable (hidden 512): router kernel + the two routed stream kernels
    "tiny": dict(n_layers=3, hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, n_experts=8, top_k=2, moe_inter=256,
                 vocab=1000, ctx_len=48),
    # one-launch MoE block applies (hidden 2048, intermediate 512); 4 query heads per KV head
    "mid": dict(n_layers=2, hidden=2048, n_heads=16, n_kv_heads=4, head_dim=128, n_experts=16, top_k=4, moe_inter=512,
                vocab=2048, ctx_len=64),
}


@pytest.fixture(params=[False, True], ids=["plain", "pdl"])
def pdl(request, K):
    """Every decode test runs with plain launches and with programmatic dependent launch."""
    prev = K.mb200_set_pdl(request.param)
    yield request.param
    K.mb200_set_pdl(prev)


@pytest.mark.parametrize("shape", ["tiny", "mid"])
def test_layers_and_logits_match_oracle(K, shape, pdl):
    from mnemocuda_b200.decode import DecodeConfig, ResidentModel
    cfg = DecodeConfig(**SHAPES[shape])
    pos0 = cfg.ctx_len - 5
    model = ResidentModel(cfg, "cuda", seed=7, kv_prefill=pos0, norm_weights="random")
    Ls = [host_layer(model, l) for l in range(cfg.n_layers)]
    kv = [(model.layers[l]["kv_k"].cpu().numpy().view(np.uint16).copy(), model.layers[l]["kv_v"].cpu().numpy().view(np.uint16).copy())
          for l in range(cfg.n_layers)]
    token = 17
    model.set_state(token, pos0)
    model.begin()
    h_gpu = model.hidden.cpu().numpy()
    assert np.array_equal(h_gpu, oracle.embedding_q4k(model.token_embd.cpu().numpy(), token, cfg.hidden))
    for l in range(cfg.n_layers):
        want, ids = oracle.decode_layer(h_gpu, Ls[l], cfg_dict(cfg), pos0, kv[l][0], kv[l][1])  # teacher forcing
        model.layer(l)
        h_gpu = model.hidden.cpu().numpy()
        rel = np.linalg.norm(h_gpu.astype(np.float64) - want) / np.linalg.norm(want)
        assert rel <= 1e-3, (l, rel)
        # the layer stored this position's K / V (fp16) where the oracle did
        gk = model.layers[l]["kv_k"].cpu().numpy().view(np.uint16)[pos0].reshape(-1)
        gv = model.layers[l]["kv_v"].cpu().numpy().view(np.uint16)[pos0].reshape(-1)
        wk = kv[l][0].reshape(cfg.ctx_len, -1)[pos0]
        wv = kv[l][1].reshape(cfg.ctx_len, -1)[pos0]
        for g_, w_ in ((gk, wk), (gv, wv)):
            a, b = g_.view(np.float16).astype(np.float64), w_.view(np.float16).astype(np.float64)
            assert np.linalg.norm(a - b) <= 2e-3 * np.linalg.norm(b)
    model.finish()
    torch.cuda.synchronize()
    normed = oracle.rms_norm(h_gpu, model.output_norm.cpu().numpy(), cfg.rms_eps)
    logits = oracle.matvec_q6k(model.lm_head.cpu().numpy(), normed, cfg.vocab, cfg.hidden)
    got = model.logits.cpu().numpy()
    assert np.linalg.norm(got - logits) <= 1e-3 * np.linalg.norm(logits)
    assert int(model.token.item()) == oracle.argmax(got)
    assert int(model.pos.item()) == pos0 + 1


def test_greedy_tokens_match_oracle_and_graph_replay(K, pdl):
    from mnemocuda_b200.decode import DecodeConfig, ResidentModel
    cfg = DecodeConfig(**SHAPES["tiny"])
    pos0, n_tok, tok0 = 20, 6, 3
    model = ResidentModel(cfg, "cuda", seed=9, kv_prefill=pos0, norm_weights="random")
    Ls = [host_layer(model, l) for l in range(cfg.n_layers)]
    kv0 = [(model.layers[l]["kv_k"].clone(), model.layers[l]["kv_v"].clone()) for l in range(cfg.n_layers)]
    kv = [(a.cpu().numpy().view(np.uint16).copy(), b.cpu().numpy().view(np.uint16).copy()) for a, b in kv0]
    # oracle
    want, t = [], tok0
    for i in range(n_tok):
        t, logits, _ = oracle_token(model, Ls, kv, t, pos0 + i)
        srt = np.sort(logits)
        assert srt[-1] - srt[-2] > 1e-3 * np.abs(srt[-1]), "near-tie in the oracle's logits: pick another seed"
        want.append(t)
    # eager
    model.set_state(tok0, pos0)
    eager = []
    for i in range(n_tok):
        model.step()
        eager.append(int(model.token.item()))
    assert eager == want
    assert int(model.pos.item()) == pos0 + n_tok
    # CUDA graph of one token, replayed: same tokens, nothing patched between replays
    for l in range(cfg.n_layers):
        model.layers[l]["kv_k"].copy_(kv0[l][0])
        model.layers[l]["kv_v"].copy_(kv0[l][1])
    model.set_state(tok0, pos0)
    g = model.capture(1)
    for l in range(cfg.n_layers):  # capture() ran one eager token: restore the cache rows it wrote
        model.layers[l]["kv_k"].copy_(kv0[l][0])
        model.layers[l]["kv_v"].copy_(kv0[l][1])
    model.set_state(tok0, pos0)
    replay = []
    for i in range(n_tok):
        g.replay()
        replay.append(int(model.token.item()))
    assert replay == want


def test_launch_overlap_does_not_change_the_tokens(K):
    """Programmatic dependent launch lets each kernel of the chain become resident before its producer has
    finished; the tokens must be those of plain launches. Buffers are reused from layer to layer with different
    contents, so a kernel that read a producer's output through a non-coherent or stale cached path would show
    here (the 30B expert shape takes the router kernel + two routed stream kernels, the 235B one the fused kernel)."""
    from mnemocuda_b200.decode import DecodeConfig, ResidentModel
    for cfg in (DecodeConfig.qwen3_30b(ctx_len=512, n_layers=6), DecodeConfig.qwen3_235b(ctx_len=512, n_layers=3)):
        cfg.vocab = 8192
        model = ResidentModel(cfg, "cuda", seed=13)
        kv0 = [(T["kv_k"].clone(), T["kv_v"].clone()) for T in model.layers]
        runs = {}
        for mode in (False, True, True):
            prev = K.mb200_set_pdl(mode)
            try:
                for T, (a, b) in zip(model.layers, kv0):
                    T["kv_k"].copy_(a)
                    T["kv_v"].copy_(b)
                model.set_state(3, cfg.ctx_len - 8)
                toks = []
                for _ in range(6):
                    model.step()
                    toks.append(int(model.token.item()))
                runs.setdefault(mode, []).append(toks)
            finally:
                K.mb200_set_pdl(prev)
        assert runs[True][0] == runs[False][0] == runs[True][1], (cfg.name, runs)
        del model
        torch.cuda.empty_cache()


def test_one_layer_at_the_235b_shape(K, pdl):
    """A single layer with the benchmark's 235B geometry (hidden 4096, 64/4 heads, 128 experts top-8,
    intermediate 1536) at the last position of an 8192-token context, against the oracle."""
    from mnemocuda_b200.decode import DecodeConfig, ResidentModel
    cfg = DecodeConfig.qwen3_235b(ctx_len=8192, n_layers=1)
    cfg.vocab = 4096  # the lm_head is not under test here
    model = ResidentModel(cfg, "cuda", seed=11)
    L = host_layer(model, 0)
    kk = model.layers[0]["kv_k"].cpu().numpy().view(np.uint16).copy()
    vv = model.layers[0]["kv_v"].cpu().numpy().view(np.uint16).copy()
    pos = cfg.ctx_len - 1
    model.set_state(5, pos)
    model.begin()
    h0 = model.hidden.cpu().numpy()
    want, ids = oracle.decode_layer(h0, L, cfg_dict(cfg), pos, kk, vv)
    for _ in range(2):  # twice from the same input: the layer leaves its counters consistent
        model.hidden.copy_(torch.from_numpy(h0).cuda())
        model.layer(0)
        got = model.hidden.cpu().numpy().astype(np.float64)
        rel = np.linalg.norm(got - want) / np.linalg.norm(want)
        assert rel <= 1e-3, rel
    assert K.mb200_device_error() == 0


def test_split_model_directory_decodes_like_the_oracle(K, pdl, tmp_path):
    """A model written in the reference's split-model layout (docs/model-format.md) with a different
    weight type on every projection, Q4_K and Q6_K down projections on alternating layers and a Q3_K
    embedding; loaded through split_model.read_split_dir and decoded: every layer and the greedy tokens
    against the oracle on the same files."""
    from mnemocuda_b200 import split_model as sm
    from mnemocuda_b200.decode import DecodeConfig
    cfg = DecodeConfig(**dict(SHAPES["tiny"], n_layers=2, ctx_len=128))
    cfg.lm_head_type = 13
    types = [(13, 8, 11, 12), (12, 12, 14, 8)]
    parts = sm.synthetic_host_model(cfg, seed=11, types=types, down_types=[12, 14], embd_type=11)
    sm.write_split_dir(str(tmp_path), cfg, *parts, embd_type=11)
    split = sm.read_split_dir(str(tmp_path))
    assert split.cfg.lm_head_type == 13 and [e.down_type for e in split.experts] == [12, 14]
    model = split.to_device("cuda")
    c = split.cfg
    Ls = [split.host_layer(l) for l in range(c.n_layers)]
    kv = [(np.zeros((c.ctx_len, c.n_kv_heads * c.head_dim), np.uint16), np.zeros((c.ctx_len, c.n_kv_heads * c.head_dim), np.uint16))
          for _ in range(c.n_layers)]

    def layer_cfg(l):
        d = cfg_dict(c)
        d["wq_type"], d["wk_type"], d["wv_type"], d["wo_type"] = Ls[l]["types"]
        d["expert_stride"], d["gate_sz"], d["up_sz"], d["down_type"] = Ls[l]["expert_layout"]
        return d

    embd, lm, onorm = split.tensor("token_embd.weight"), split.tensor("output.weight"), split.tensor("output_norm.weight")
    token, want_tokens, got_tokens = 5, [], []
    model.set_state(token, 0)
    for pos in range(4):
        h = oracle.dequant_type(11, embd, c.vocab, c.hidden)[token]
        model.begin()
        assert np.array_equal(model.hidden.cpu().numpy(), h)
        for l in range(c.n_layers):
            h, _ = oracle.decode_layer(h, Ls[l], layer_cfg(l), pos, kv[l][0], kv[l][1])
            model.layer(l)
            got = model.hidden.cpu().numpy().astype(np.float64)
            rel = np.linalg.norm(got - h) / np.linalg.norm(h)
            assert rel <= 1e-3, (pos, l, rel)
            h = got.astype(np.float32)  # teacher forcing: the next layer starts from the device's state
            kv[l][0][pos] = model.layers[l]["kv_k"].cpu().numpy().view(np.uint16)[pos].reshape(-1)
            kv[l][1][pos] = model.layers[l]["kv_v"].cpu().numpy().view(np.uint16)[pos].reshape(-1)
        model.finish()
        logits = oracle.matvec_type(13, lm, oracle.rms_norm(h, onorm, c.rms_eps), c.vocab, c.hidden)
        got_logits = model.logits.cpu().numpy()
        assert np.linalg.norm(got_logits - logits) <= 1e-3 * np.linalg.norm(logits)
        token = int(model.token.item())
        assert token == oracle.argmax(got_logits)
        assert int(model.pos.item()) == pos + 1
