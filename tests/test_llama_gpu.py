"""GPU decoder (paged KV, sm_100a kernels) against the fp32 oracle on a small head_dim-128 model."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _small_cfg(arch=None, **kw):
    from inference_b200.models import ModelConfig

    base = dict(hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
                num_key_value_heads=2, head_dim=128, vocab_size=2048, rms_norm_eps=1e-5, rope_theta=10000.0)
    base.update(kw)
    if arch:
        base["model_type"] = arch
    return ModelConfig.from_json(base)


def _build(cfg, bias=False, seed=0):
    from inference_b200.engine.kv_pool import PagedKvPool
    from inference_b200.engine.runner import ModelRunner
    from inference_b200.models.llama import LlamaGpu
    from inference_b200.models.oracle import OracleLlama, random_llama_weights

    w = random_llama_weights(cfg, seed=seed, std=0.05, bias=bias)
    w = {k: v.bfloat16().float() for k, v in w.items()}  # both models see identical bf16-representable weights
    oracle = OracleLlama(cfg, w, dtype=torch.float32, device="cuda")
    model = LlamaGpu(cfg, device=torch.device("cuda")).load_state_dict(w)
    pool = PagedKvPool(cfg.num_layers, 256, model.hkv, cfg.head_dim, 16, device="cuda")
    runner = ModelRunner(model, pool, max_batch=8, max_seq_len=512)
    return oracle, model, pool, runner


@pytest.mark.parametrize("arch,bias", [(None, False), ("qwen2", True), ("qwen3", False), ("gemma2", False),
                                       ("glm4", True), ("glm", True), ("qwen2_moe", True)])
def test_prefill_and_decode_logits_match_oracle(arch, bias):
    from inference_b200.engine.kv_pool import PagedSequence

    kw = {}
    if arch == "gemma2":
        kw = dict(attn_logit_softcapping=50.0, final_logit_softcapping=30.0, query_pre_attn_scalar=128)
    if arch in ("glm4", "glm"):
        kw = dict(partial_rotary_factor=0.5)
    if arch == "qwen2_moe":
        kw = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=256,
                  shared_expert_intermediate_size=512, norm_topk_prob=False)
    cfg = _small_cfg(arch, **kw)
    oracle, model, pool, runner = _build(cfg, bias=bias)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (37, 5, 64)]
    seqs = [PagedSequence(pool) for _ in prompts]
    logits = runner.prefill(seqs, prompts, want_logits=True)
    caches = []
    for i, p in enumerate(prompts):
        c = oracle.make_cache()
        ref = oracle.decode_logits(torch.tensor([p], device="cuda"), c, 0)[0]
        caches.append(c)
        err = (logits[i] - ref).abs().max().item()
        assert err < 0.08 * max(1.0, ref.abs().max().item()), (arch, i, err)
    # a few decode steps through the graph path
    toks = [int(logits[i].argmax()) for i in range(len(prompts))]
    for step in range(3):
        lg = runner.decode(seqs, toks, want_logits=True)
        for i in range(len(prompts)):
            ref = oracle.decode_logits(torch.tensor([[toks[i]]], device="cuda"), caches[i], caches[i].offset)[0]
            err = (lg[i] - ref).abs().max().item()
            assert err < 0.08 * max(1.0, ref.abs().max().item()), (arch, step, i, err)
        toks = [int(lg[i].argmax()) for i in range(len(prompts))]


def test_greedy_decode_matches_oracle_tokens():
    from inference_b200.engine.kv_pool import PagedSequence

    cfg = _small_cfg()
    oracle, model, pool, runner = _build(cfg, seed=3)
    prompt = torch.randint(0, cfg.vocab_size, (16,), generator=torch.Generator().manual_seed(0)).tolist()
    ref_tokens, margins = oracle.generate_greedy(prompt, 24)
    seq = PagedSequence(pool)
    tok = int(runner.prefill([seq], [prompt])[0])
    got = [tok]
    for _ in range(23):
        tok = int(runner.decode([seq], [tok])[0])
        got.append(tok)
    for i, (a, b) in enumerate(zip(got, ref_tokens)):
        if a != b:
            assert margins[i] < 0.05, f"diverged at step {i} with margin {margins[i]}"
            break


@pytest.mark.parametrize("fmt", ["Q4_K", "Q8_0"])
def test_quantised_model_matches_oracle_on_dequantised_weights(fmt):
    """quantize_() swaps the projections for packed weights; logits must match the fp32 oracle run on the very
    weights those packed bytes decode to (prefill uses the expand + dense GEMM path, decode the fused dequant-GEMM)."""
    from inference_b200.engine.kv_pool import PagedKvPool, PagedSequence
    from inference_b200.engine.runner import ModelRunner
    from inference_b200.models.llama import LlamaGpu
    from inference_b200.models.oracle import OracleLlama, random_llama_weights
    from inference_b200.ops import quant

    cfg = _small_cfg()
    w = {k: v.bfloat16().float() for k, v in random_llama_weights(cfg, seed=2, std=0.05).items()}
    proj = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
    wq = {k: (quant.dequantize_reference(quant.quantize_on_device(v, fmt)) if any(p in k for p in proj) else v)
          for k, v in w.items()}
    oracle = OracleLlama(cfg, wq, dtype=torch.float32, device="cuda")
    model = LlamaGpu(cfg, device=torch.device("cuda")).load_state_dict(w).quantize_(fmt)
    assert model.quant_format == fmt and not isinstance(model.layers[0].qkv, torch.Tensor)
    pool = PagedKvPool(cfg.num_layers, 256, model.hkv, cfg.head_dim, 16, device="cuda")
    runner = ModelRunner(model, pool, max_batch=4, max_seq_len=512)
    prompts = [list(range(5, 90)), list(range(300, 312))]
    seqs = [PagedSequence(pool) for _ in prompts]
    logits = runner.prefill(seqs, prompts, want_logits=True)
    caches = []
    for i, p in enumerate(prompts):
        c = oracle.make_cache()
        ref = oracle.decode_logits(torch.tensor([p], device="cuda"), c, 0)[0]
        caches.append(c)
        assert (logits[i] - ref).abs().max().item() < 0.1 * max(1.0, ref.abs().max().item())
    toks = [int(logits[i].argmax()) for i in range(2)]
    for step in range(3):
        lg = runner.decode(seqs, toks, want_logits=True)
        for i in range(2):
            ref = oracle.decode_logits(torch.tensor([[toks[i]]], device="cuda"), caches[i], caches[i].offset)[0]
            assert (lg[i] - ref).abs().max().item() < 0.1 * max(1.0, ref.abs().max().item()), (fmt, step, i)
        toks = [int(lg[i].argmax()) for i in range(2)]


def test_padded_decode_buckets_reuse_graphs_and_match_exact_batches():
    """Decode batches padded to a graph bucket produce the tokens of the unpadded eager step, and a job
    whose batch shrinks one lane at a time captures one graph per bucket, not one per batch size."""
    from inference_b200.engine.kv_pool import PagedKvPool, PagedSequence
    from inference_b200.engine.runner import ModelRunner, _bucket

    assert [_bucket(b, 128) for b in (1, 8, 9, 16, 17, 64, 65, 127)] == [1, 8, 16, 16, 24, 64, 80, 128]
    cfg = _small_cfg()
    _, model, _, _ = _build(cfg, seed=5)
    outs = []
    for padded in (True, False):
        pool = PagedKvPool(cfg.num_layers, 512, model.hkv, cfg.head_dim, 16, device="cuda")
        runner = ModelRunner(model, pool, max_batch=32, max_seq_len=256, use_graphs=padded)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg.vocab_size, (5 + 3 * i,), generator=g).tolist() for i in range(13)]
        seqs = [PagedSequence(pool) for _ in prompts]
        toks = runner.prefill(seqs, prompts).tolist()
        trace = []
        for step in range(6):
            toks = runner.decode(seqs, toks).tolist()
            trace.append(list(toks))
            seqs, toks = seqs[:-1], toks[:-1]       # one lane finishes per step: 13, 12, ..., 8 live rows
        outs.append(trace)
        if padded:
            assert runner.captures == 2             # buckets 16 and 8
    assert outs[0] == outs[1]


def test_prefill_embedding_override_matches_oracle_with_spliced_embeds():
    """Rows whose embeddings are replaced (image features of a vision-language prompt) flow through the GPU
    prefill exactly like the oracle's forward on spliced embeddings; decoding continues from the paged cache."""
    from inference_b200.engine.kv_pool import PagedSequence
    from inference_b200.media.vision_providers import EngineLm, OracleLm

    cfg = _small_cfg()
    oracle, model, pool, runner = _build(cfg, seed=9)
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, cfg.vocab_size, (12,), generator=g).tolist()
    pos = [2, 3, 4, 5]
    feats = (torch.randn(4, cfg.hidden_size, generator=g) * 0.05).bfloat16().float()
    seq = PagedSequence(pool)
    logits = runner.prefill([seq], [ids], want_logits=True, embed_overrides=[(pos, feats.cuda())])[0]
    emb = oracle.embed(torch.tensor([ids], device="cuda")).clone()
    emb[0, pos] = feats.cuda()
    cache = oracle.make_cache()
    ref = oracle.project_logits(oracle.hidden_states(None, cache, 0, embeds=emb)[:, -1:, :])[0, 0]
    assert (logits - ref).abs().max().item() < 0.05 * max(1.0, ref.abs().max().item())
    plain = runner.prefill([PagedSequence(pool)], [ids], want_logits=True)[0]
    assert (plain - logits).abs().max().item() > 1e-3           # the override changed the result
    seq.release()

    class _Eng:
        def __init__(s):
            s.runner = runner

        def new_sequence(s):
            return PagedSequence(pool)
    got = EngineLm(_Eng()).generate_with_embeds(ids, pos, feats.cuda(), 8)
    want = OracleLm(oracle).generate_with_embeds(ids, pos, feats, 8)
    agree = sum(a == b for a, b in zip(got, want))
    assert len(got) == 8 and agree >= 6, (got, want)


def test_pipeline_sharded_stages_match_the_single_model(monkeypatch):
    """Two pipeline stages (both placed on this GPU) hand the residual stream across the boundary and reproduce
    the unsharded model's logits for prefill and paged decode (bit-identical with the folded-norm decode chain off:
    a stage boundary restarts the chain with a norm kernel, which rounds differently)."""
    monkeypatch.setenv("SWB_NORM_CHAIN", "0")
    from inference_b200.engine.kv_pool import PagedSequence
    from inference_b200.engine.llm_engine import EngineConfig, LlmEngine
    from inference_b200.models.llama import LlamaGpu
    from inference_b200.models.oracle import random_llama_weights
    from inference_b200.models.pipeline import PipelineLlama

    cfg = _small_cfg()
    w = {k: v.bfloat16().float() for k, v in random_llama_weights(cfg, seed=4, std=0.05).items()}
    single = LlmEngine(LlamaGpu(cfg, device=torch.device("cuda")).load_state_dict(w),
                       EngineConfig(max_batch=4, max_seq_len=256, use_graphs=False))
    pipe_model = PipelineLlama(cfg, ["cuda:0", "cuda:0"]).load_state_dict(w)
    assert [len(b) for b in pipe_model.blocks] == [2, 1] and len(pipe_model.layer_devices()) == 3
    assert pipe_model.stages[0].lm_head is None and pipe_model.stages[1].embed is None
    pipe = LlmEngine(pipe_model, EngineConfig(max_batch=4, max_seq_len=256))
    assert not pipe.runner.use_graphs and len(pipe.pool.data) == 2
    prompts = [list(range(3, 40)), list(range(100, 109))]
    outs = []
    for eng in (single, pipe):
        seqs = [eng.new_sequence() for _ in prompts]
        lg = eng.runner.prefill(seqs, prompts, want_logits=True)
        toks = [int(lg[i].argmax()) for i in range(2)]
        steps = [lg]
        for _ in range(3):
            lg = eng.runner.decode(seqs, toks, want_logits=True)
            steps.append(lg.clone())
            toks = [int(lg[i].argmax()) for i in range(2)]
        outs.append(steps)
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_pipeline_sharded_across_two_gpus_matches_single_gpu(monkeypatch):
    monkeypatch.setenv("SWB_NORM_CHAIN", "0")
    from inference_b200.engine.llm_engine import EngineConfig, LlmEngine
    from inference_b200.models.llama import LlamaGpu
    from inference_b200.models.oracle import random_llama_weights
    from inference_b200.models.pipeline import PipelineLlama

    cfg = _small_cfg()
    w = {k: v.bfloat16().float() for k, v in random_llama_weights(cfg, seed=6, std=0.05).items()}
    single = LlmEngine(LlamaGpu(cfg, device=torch.device("cuda:0")).load_state_dict(w),
                       EngineConfig(max_batch=2, max_seq_len=128, use_graphs=False))
    pipe = LlmEngine(PipelineLlama(cfg, ["cuda:0", "cuda:1"]).load_state_dict(w), EngineConfig(max_batch=2, max_seq_len=128))
    assert pipe.model.stages[1].layers[0].qkv.device.index == 1 and all(b > 0 for b in pipe.model.weight_bytes())
    prompt = [list(range(7, 50))]
    outs = []
    for eng in (single, pipe):
        seqs = [eng.new_sequence()]
        lg = eng.runner.prefill(seqs, prompt, want_logits=True)
        tok = [int(lg[0].argmax())]
        trace = [lg.cpu()]
        for _ in range(3):
            lg = eng.runner.decode(seqs, tok, want_logits=True)
            trace.append(lg.cpu().clone())
            tok = [int(lg[0].argmax())]
        outs.append(trace)
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("arch,bias", [(None, False), ("qwen2", True), ("qwen3", False)])
def test_folded_norm_decode_chain_matches_oracle_with_non_unit_norm_weights(arch, bias, monkeypatch):
    """Decode steps of an unsharded dense model skip the norm kernels (norm weights folded into qkv / gate_up, 1 / rms
    applied in the GEMM epilogues from the sums of squares the o / down epilogues emit). Checked with random norm
    weights against the oracle, against the un-folded model, and for determinism."""
    from inference_b200.engine.kv_pool import PagedKvPool, PagedSequence
    from inference_b200.engine.runner import ModelRunner
    from inference_b200.models.llama import LlamaGpu
    from inference_b200.models.oracle import OracleLlama, random_llama_weights

    cfg = _small_cfg(arch)
    g = torch.Generator().manual_seed(11)
    w = random_llama_weights(cfg, seed=7, std=0.05, bias=bias)
    for k in w:
        if k.endswith("layernorm.weight") or k == "model.norm.weight":
            w[k] = 0.5 + torch.rand(w[k].shape, generator=g)
    w = {k: v.bfloat16().float() for k, v in w.items()}
    oracle = OracleLlama(cfg, w, dtype=torch.float32, device="cuda")
    prompts = [list(range(5, 40)), list(range(300, 309)), list(range(50, 71))]

    def run(fold: str):
        monkeypatch.setenv("SWB_FOLD_NORMS", fold)
        model = LlamaGpu(cfg, device=torch.device("cuda")).load_state_dict(w)
        assert model.norm_folded == (fold == "1") and model._chain_ok == (fold == "1")
        pool = PagedKvPool(cfg.num_layers, 256, model.hkv, cfg.head_dim, 16, device="cuda")
        runner = ModelRunner(model, pool, max_batch=8, max_seq_len=512)
        seqs = [PagedSequence(pool) for _ in prompts]
        lg = runner.prefill(seqs, prompts, want_logits=True)
        trace = [lg.clone()]
        toks = [int(lg[i].argmax()) for i in range(len(prompts))]
        for _ in range(4):
            lg = runner.decode(seqs, toks, want_logits=True)
            trace.append(lg.clone())
            toks = [int(lg[i].argmax()) for i in range(len(prompts))]
        return trace, model

    folded, model = run("1")
    plain, _ = run("0")
    assert model.launches == 1 + cfg.num_layers * 6 + 1 + 1 + 1   # embedding, 6 per layer, first-layer norm, final norm, head
    again, _ = run("1")
    for a, b in zip(folded, again):
        assert torch.equal(a, b)                                    # fixed reduction order: bit-identical reruns
    caches = []
    for i, p in enumerate(prompts):
        c = oracle.make_cache()
        ref = oracle.decode_logits(torch.tensor([p], device="cuda"), c, 0)[0]
        caches.append(c)
        assert (folded[0][i] - ref).abs().max().item() < 0.05 * max(1.0, ref.abs().max().item())
    toks = [int(folded[0][i].argmax()) for i in range(len(prompts))]
    for step in range(1, 5):
        for i in range(len(prompts)):
            ref = oracle.decode_logits(torch.tensor([[toks[i]]], device="cuda"), caches[i], caches[i].offset)[0]
            scale = max(1.0, ref.abs().max().item())
            assert (folded[step][i] - ref).abs().max().item() < 0.05 * scale, (step, i)
        toks = [int(folded[step][i].argmax()) for i in range(len(prompts))]
    # the un-folded model fed the same tokens agrees (its own greedy history may branch at near-ties, so only the
    # prefill and the first decode step, whose inputs are provably identical, are compared)
    for step in (0, 1):
        same = [int(folded[0][i].argmax()) == int(plain[0][i].argmax()) for i in range(len(prompts))]
        for i in range(len(prompts)):
            if step == 0 or same[i]:
                d = (folded[step][i] - plain[step][i]).abs().max().item()
                assert d < 0.05 * max(1.0, plain[step][i].abs().max().item()), (step, i, d)


def test_qwen3_vl_provider_on_the_device(tmp_path):
    """The vision-language provider of the sm_100a bundle: tower and decoder in bf16 on the device; an image prompt
    decodes, and the tower's tokens track the fp32 tower."""
    import json
    import sys
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).parent))
    from test_qwen3_vl_cpu import _hf

    import inference_b200.models.qwen3_vl as Q3
    from inference_b200.bundles import runtime_b200
    from inference_b200.contracts.core_llm import LoadSpec, Message, Role, TextLlmRequest
    from inference_b200.contracts.core_llm.message import ImageRef, Text
    from inference_b200.contracts.core_llm.request import Sampling
    from inference_b200.io.safetensors_io import save_file
    from inference_b200.testkit.synthetic import wordlevel_tokenizer_json

    cfg, hf = _hf(seed=5)
    top = cfg.to_dict()
    top["model_type"], top["architectures"] = "qwen3_vl", ["Qwen3VLForConditionalGeneration"]
    (tmp_path / "config.json").write_text(json.dumps(top))
    sd = {k: v.contiguous() for k, v in hf.state_dict().items()}
    save_file(sd, tmp_path / "model.safetensors")
    tok = json.loads(wordlevel_tokenizer_json(200))
    special = {150: "<|image_pad|>", 151: "<|video_pad|>", 152: "<|vision_start|>", 153: "<|vision_end|>"}
    tok["model"]["vocab"] = {special.get(i, w): i for w, i in tok["model"]["vocab"].items()}
    tok["added_tokens"] = tok.get("added_tokens", []) + [
        {"id": i, "content": c, "single_word": False, "lstrip": False, "rstrip": False, "normalized": False, "special": True}
        for i, c in special.items()]
    (tmp_path / "tokenizer.json").write_text(json.dumps(tok))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"eos_token": "<|im_end|>"}))
    llm = runtime_b200.catalog().text().load_for_model(LoadSpec.dense(str(tmp_path)))
    assert llm.descriptor().id == "b200-qwen3-vl"
    vc = Q3.Qwen3VlVisionConfig.from_json(top)
    patches = torch.randn(24, vc.patch_dim, generator=torch.Generator().manual_seed(4))
    ref, _ = Q3.Qwen3VlVisionTower(vc, sd).forward(patches, [(1, 4, 6)])
    out, taps = llm.tower.forward(patches, [(1, 4, 6)])
    assert out.is_cuda and len(taps) == 3
    assert (out.float().cpu() - ref).abs().max().item() < 0.08 * max(1.0, ref.abs().max().item())
    g = torch.Generator().manual_seed(5)
    raw = bytes(torch.randint(0, 256, (16 * 24 * 3,), generator=g, dtype=torch.uint8).tolist())
    req = TextLlmRequest(messages=[Message(Role.USER, [ImageRef(24, 16, raw), Text("the cat sat")])], max_new_tokens=4,
                         seed=0, sampling=Sampling(temperature=0.0))
    orig = Q3.image_to_patches                    # this tiny tower has 4-pixel patches: keep the image at its own size
    Q3.image_to_patches = lambda rgb, vc_, **kw: orig(rgb, vc_, min_pixels=16, max_pixels=10 ** 6)
    try:
        res = llm.generate(req, on_event=lambda e: None)
    finally:
        Q3.image_to_patches = orig
    assert res.usage.generated_tokens >= 1


def test_qwen3_vl_paged_decoder_matches_the_oracle_decoder(tmp_path, monkeypatch):
    """Qwen3-VL with 128-wide heads runs on the paged sm_100a decoder: the image prompt's three-axis rotary table and
    DeepStack taps ride on the prefill step, later tokens continue at the shifted position. Same snapshot and request
    through the oracle decoder (bf16, framework ops): the first-step logits agree and greedy decoding emits the same
    tokens; a text-only request on the same provider still decodes."""
    import json
    import sys
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).parent))
    from test_qwen3_vl_cpu import _hf

    import inference_b200.models.qwen3_vl as Q3
    from inference_b200.bundles import runtime_b200
    from inference_b200.contracts.core_llm import LoadSpec, Message, Role, TextLlmRequest
    from inference_b200.contracts.core_llm.message import ImageRef, Text
    from inference_b200.contracts.core_llm.request import Sampling
    from inference_b200.engine.backend import GpuBackend, OracleBackend
    from inference_b200.io.safetensors_io import save_file
    from inference_b200.testkit.synthetic import wordlevel_tokenizer_json

    cfg, hf = _hf(seed=5, head_dim=128, mrope_section=(24, 20, 20))
    top = cfg.to_dict()
    top["model_type"], top["architectures"] = "qwen3_vl", ["Qwen3VLForConditionalGeneration"]
    (tmp_path / "config.json").write_text(json.dumps(top))
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, tmp_path / "model.safetensors")
    tok = json.loads(wordlevel_tokenizer_json(200))
    special = {150: "<|image_pad|>", 151: "<|video_pad|>", 152: "<|vision_start|>", 153: "<|vision_end|>"}
    tok["model"]["vocab"] = {special.get(i, w): i for w, i in tok["model"]["vocab"].items()}
    tok["added_tokens"] = tok.get("added_tokens", []) + [
        {"id": i, "content": c, "single_word": False, "lstrip": False, "rstrip": False, "normalized": False, "special": True}
        for i, c in special.items()]
    (tmp_path / "tokenizer.json").write_text(json.dumps(tok))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"eos_token": "<|im_end|>"}))
    g = torch.Generator().manual_seed(5)
    raw = bytes(torch.randint(0, 256, (16 * 24 * 3,), generator=g, dtype=torch.uint8).tolist())
    req = lambda: TextLlmRequest(messages=[Message(Role.USER, [ImageRef(24, 16, raw), Text("the cat sat on the mat")])],   # noqa: E731
                                 max_new_tokens=6, seed=0, sampling=Sampling(temperature=0.0))
    orig = Q3.image_to_patches
    monkeypatch.setattr(Q3, "image_to_patches", lambda rgb, vc_, **kw: orig(rgb, vc_, min_pixels=16, max_pixels=10 ** 6))
    out, first = {}, {}
    for mode, kind in (("paged", GpuBackend), ("oracle", OracleBackend)):
        monkeypatch.setenv("SWB_QWEN3_VL_DECODER", mode)
        llm = runtime_b200.catalog().text().load_for_model(LoadSpec.dense(str(tmp_path)))
        assert isinstance(llm.backend, kind), mode
        r = req()
        res = llm.generate(r, on_event=lambda e: None)
        out[mode] = res.text
        assert res.usage.generated_tokens >= 1
        # first-step logits through the backend itself
        prompt_ids, seq = llm._splice_media(r, _prompt_ids(llm, r))
        first[mode] = llm.backend.forward([seq], [prompt_ids])[0].float().cpu()
        nxt = int(first[mode].argmax())
        second = llm.backend.forward([seq], [[nxt]])[0].float().cpu()       # the decode step continues at the shifted position
        first[mode + "2"] = second
        llm.backend.release(seq)
        if mode == "paged":
            plain = llm.generate(TextLlmRequest(messages=[Message(Role.USER, [Text("the cat sat")])], max_new_tokens=3, seed=0,
                                                sampling=Sampling(temperature=0.0)), on_event=lambda e: None)
            assert plain.usage.generated_tokens >= 1
        del llm
    for k in ("paged", "paged2"):
        ref = first[k.replace("paged", "oracle")]
        assert (first[k] - ref).abs().max().item() < 0.06 * max(1.0, ref.abs().max().item()), k
    assert out["paged"] == out["oracle"]


def _prompt_ids(llm, req):
    """The provider's own prompt rendering, without running a generation."""
    from inference_b200.contracts.core_llm import RenderOptions

    prompt = llm.template.render_with(llm._render_messages(req), RenderOptions(True, req.enable_thinking_kwarg(), req.tools))
    return llm.tokenizer.encode(prompt, add_special_tokens=False)


def test_split_decode_steps_match_whole_steps():
    """A decode batch run as consecutive sub-steps of at most `decode_split` rows (the knob that keeps a
    large batch inside the row limit of the chained path) gives the logits of the whole-batch step, with
    and without graphs, and leaves the caches in the same state for the following step."""
    from inference_b200.engine.kv_pool import PagedKvPool, PagedSequence
    from inference_b200.engine.runner import ModelRunner

    cfg = _small_cfg()
    _, model, _, _ = _build(cfg, seed=6)
    outs = []
    for split, graphs in ((0, False), (4, False), (4, True)):
        pool = PagedKvPool(cfg.num_layers, 512, model.hkv, cfg.head_dim, 16, device="cuda")
        runner = ModelRunner(model, pool, max_batch=32, max_seq_len=256, use_graphs=graphs)
        runner.decode_split = split
        g = torch.Generator().manual_seed(2)
        prompts = [torch.randint(0, cfg.vocab_size, (4 + 2 * i,), generator=g).tolist() for i in range(11)]
        seqs = [PagedSequence(pool) for _ in prompts]
        toks = runner.prefill(seqs, prompts).tolist()
        steps = []
        for _ in range(3):
            lg = runner.decode(seqs, toks, want_logits=True).float().clone()
            steps.append(lg.cpu())
            toks = outs[0][1][len(steps) - 1] if outs else lg.argmax(-1).tolist()
        outs.append((steps, [s.argmax(-1).tolist() for s in steps]))
    ref = outs[0][0]
    for steps, _ in outs[1:]:
        for a, b in zip(steps, ref):
            assert a.shape == b.shape
            assert (a - b).abs().max().item() < 0.03 * max(1.0, b.abs().max().item())
