"""MOSS-TTS-Realtime: configuration checks, the sampler, prompt and turn layouts, cached against uncached backbone steps,
the depth transformer against a cache-free restatement, the codec stages against an explicit-softmax restatement and its
causality (what streaming relies on), chunked streaming, and the generator: conformance, streaming, voice clone, and the
equality of a conversation rendered in one request and turn by turn through a session."""
import json
import math

import pytest
import torch
import torch.nn.functional as F

from inference_b200.audio import moss_tts_realtime as M
from inference_b200.audio.moss_ttsd import Rng


@pytest.fixture(scope="module")
def snap(tmp_path_factory):
    return M.write_synthetic_snapshot(tmp_path_factory.mktemp("mtr") / "model")


@pytest.fixture(scope="module")
def loaded(snap):
    import tokenizers

    from inference_b200.io.safetensors_io import load_file

    cfg = M.RealtimeConfig.from_json(json.loads((snap[0] / "config.json").read_text()))
    return M.Decoder(cfg, load_file(snap[0] / M.MODEL_WEIGHTS)), tokenizers.Tokenizer.from_file(str(snap[0] / "tokenizer.json")), cfg


def test_config_checks(snap):
    from inference_b200.contracts.errors import LoadError

    j = json.loads((snap[0] / "config.json").read_text())
    cfg = M.RealtimeConfig.from_json(j)
    assert (cfg.rvq, cfg.audio_pad_token, cfg.audio_bos, cfg.audio_eos) == (4, 8, 9, 10)
    real = M.RealtimeConfig.from_json({"rvq": 16, "audio_vocab_size": 1027, "audio_pad_token": 1024, "language_config": {},
                                       "local_config": {"rvq": 16}})
    assert (real.audio_bos, real.audio_eos, real.text_pad, real.reference_audio_pad) == (1025, 1026, 151_655, 151_654)
    for bad in ({"rvq": 8}, {"rvq": 0, "local_config": {**j["local_config"], "rvq": 0}}, {"audio_vocab_size": 10}):
        with pytest.raises(LoadError):
            M.RealtimeConfig.from_json({**j, **bad})
    with pytest.raises(LoadError):
        M.RealtimeConfig.from_json({k: v for k, v in j.items() if k != "local_config"})


def test_sampler(monkeypatch):
    p = M.SamplingParams()
    assert (p.temperature, p.top_p, p.top_k, p.repetition_penalty, p.repetition_window) == (0.8, 0.6, 30, 1.1, 50)
    a, b = Rng(42), Rng(42)
    assert [a.next_f32() for _ in range(8)] == [b.next_f32() for _ in range(8)]
    greedy = M.SamplingParams(temperature=0.0)
    assert M.sample(torch.tensor([0.1, 5.0, 0.2, -1.0]), [], greedy, Rng(1)) == 1
    top1 = M.SamplingParams(1.0, 1.0, 1, 1.0)
    assert all(M.sample(torch.tensor([1.0, 2.0, 9.0, 3.0, 0.5]), [], top1, Rng(s)) == 2 for s in range(10))
    # the penalty divides positive logits and multiplies negative ones, only for tokens inside the window
    strong = M.SamplingParams(temperature=0.0, repetition_penalty=2.0, repetition_window=2)
    lg = torch.tensor([4.0, 3.0, -1.0])
    assert M.sample(lg, [0], strong, Rng(0)) == 1                  # 4 / 2 < 3
    assert M.sample(lg, [0, 2, 2], strong, Rng(0)) == 0            # token 0 fell out of the 2-token window
    assert M.sample(torch.tensor([-1.0, -1.5]), [0], strong, Rng(0)) == 1     # -1 * 2 < -1.5
    assert torch.equal(lg, torch.tensor([4.0, 3.0, -1.0]))        # the caller's logits are untouched
    monkeypatch.setenv("MOSS_TTS_TEMPERATURE", "0.5")
    monkeypatch.setenv("MOSS_TTS_TOP_K", "7")
    monkeypatch.setenv("MOSS_TTS_TOP_P", "nan")
    e = M.SamplingParams.from_env()
    assert (e.temperature, e.top_k, e.top_p) == (0.5, 7, 0.6)
    monkeypatch.setenv("MOSS_TTS_MIN_FRAMES", "40")
    assert M.min_eos_frames(20) == 10 and M.min_eos_frames(200) == 40
    assert M.turn_seed(5, 0) == 5 and M.turn_seed(5, 1) != M.turn_seed(5, 2)


def test_prompt_and_turn_layouts(loaded):
    from inference_b200.contracts.errors import InferenceError

    _, tok, cfg = loaded
    ids = lambda s: tok.encode(s, add_special_tokens=False).ids                       # noqa: E731
    plain = M.system_frames(tok, cfg, None)
    assert [f[0] for f in plain] == ids(M.TTS_SYSTEM_PROMPT) and all(f[1:] == [cfg.audio_pad_token] * 4 for f in plain)
    ref = [[1, 2, 3, 4], [5, 6, 7, 0], [2, 2, 2, 2]]
    cloned = M.system_frames(tok, cfg, ref)
    carried = [f[1:] for f in cloned if f[0] == cfg.reference_audio_pad]
    assert carried == ref and len(cloned) > len(plain)
    with pytest.raises(InferenceError):
        M.system_frames(tok, cfg, [[1, 2, 3]])
    # assistant: opener + the first 12 text tokens, the begin token on the last prefilled position, the rest streams
    text = "hello there how are you fine thanks and you hello there how are you"
    n = len(ids(text))
    assert n > M.DELAY_TOKENS_LEN
    frames = []
    streamed = M.assistant_prefill(tok, cfg, M.ASSISTANT_OPEN, text, frames)
    assert len(frames) == len(ids(M.ASSISTANT_OPEN)) + 12 and streamed == ids(text)[12:]
    assert frames[-1][1] == cfg.audio_bos and all(f[1] == cfg.audio_pad_token for f in frames[:-1])
    short = []
    assert M.assistant_prefill(tok, cfg, M.ASSISTANT_OPEN, "hello", short) == [] and short[-1][1] == cfg.audio_bos
    with pytest.raises(InferenceError):
        M.assistant_prefill(tok, cfg, M.ASSISTANT_OPEN, "", [])
    # user turn, long text: audio starts 12 tokens into the text; begin before it, end after it
    codes = [[(i + c) % 8 for c in range(4)] for i in range(5)]
    body = M.user_body_frames(tok, cfg, text, codes)
    at = len(ids(M.USER_OPEN)) + 12
    assert [f[1:] for f in body[at:at + 5]] == codes and body[at - 1][1] == cfg.audio_bos and body[at + 5][1] == cfg.audio_eos
    assert len(body) == len(ids(M.USER_OPEN)) + n + (5 + 12 - n + 1) if 5 + 12 - n + 1 > 0 else True
    # short text: the audio sits at the end of the body
    body = M.user_body_frames(tok, cfg, "hello", codes)
    assert [f[1:] for f in body[-6:-1]] == codes and body[-1][1] == cfg.audio_eos and body[-7][1] == cfg.audio_bos
    assert all(f[0] == cfg.text_pad for f in body[-6:])
    for bad in ((text, []), ("", codes), (text, [[1, 2]])):
        with pytest.raises(InferenceError):
            M.user_body_frames(tok, cfg, *bad)


def test_backbone_cached_steps_match_one_pass(loaded):
    dec, _, cfg = loaded
    g = torch.Generator().manual_seed(0)
    frames = [[int(torch.randint(0, 300, (1,), generator=g))] + torch.randint(0, 11, (4,), generator=g).tolist() for _ in range(7)]
    whole = dec.backbone.forward(frames, dec.backbone.new_cache())
    cache = dec.backbone.new_cache()
    dec.backbone.forward(frames[:4], cache)
    for f in frames[4:6]:
        dec.backbone.forward([f], cache)
    last = dec.backbone.forward([frames[6]], cache)
    assert cache.offset == 7 and last.shape == (1, 1, 32)
    assert torch.allclose(last, whole, atol=1e-5)
    e = dec.backbone.embed(frames[:1])[0, 0]
    want = sum(dec.backbone.tables[c][frames[0][c]] for c in range(5))
    assert torch.allclose(e, want)


def test_depth_transformer_matches_cache_free_restatement(loaded, monkeypatch):
    dec, _, cfg = loaded
    local = dec.local
    hidden = torch.randn(1, 1, 32, generator=torch.Generator().manual_seed(3))
    greedy = M.SamplingParams(temperature=0.0, repetition_penalty=1.0)
    got = local.decode_frame(hidden, [], greedy, Rng(0), False)
    # restatement: re-run the whole depth sequence without a cache for every codebook
    from inference_b200.models.oracle import ContiguousKvCache
    seq, want = hidden.clone(), []
    for i in range(cfg.rvq):
        h = local.lm._norm(local.lm.hidden_states(None, ContiguousKvCache(local.layers), 0, embeds=seq)[:, -1], "model.norm.weight")
        tok = int((h @ local.heads[i].t()).argmax())
        want.append(tok)
        if i + 1 < cfg.rvq:
            seq = torch.cat([seq, local.tables[i][tok][None, None]], dim=1)
    assert got == want and len(got) == 4
    # suppression removes the end token from codebook 0 only
    seen = local.lm._norm(local.lm.hidden_states(None, ContiguousKvCache(local.layers), 0, embeds=hidden)[:, -1], "model.norm.weight")[0]
    forced = torch.zeros_like(local.heads[0])
    forced[cfg.audio_eos] = 50.0 * seen / seen.norm()           # head 0 now puts everything on the end token
    monkeypatch.setattr(local, "heads", [forced] + local.heads[1:])
    assert local.decode_frame(hidden, [], greedy, Rng(0), False)[0] == cfg.audio_eos
    assert local.decode_frame(hidden, [], greedy, Rng(0), True)[0] != cfg.audio_eos
    # sampled frames are reproducible per seed and differ across seeds
    monkeypatch.undo()
    soft = M.SamplingParams(temperature=1.5, top_p=1.0)
    a = [local.decode_frame(hidden, [], soft, Rng(s), True) for s in (1, 1, 2, 3, 4)]
    assert a[0] == a[1] and len({tuple(x) for x in a}) > 1


def test_generate_and_replay(loaded, monkeypatch):
    dec, tok, cfg = loaded
    monkeypatch.setattr(M, "min_eos_frames", lambda budget: budget)          # never stop early: the toy model has no notion of an end
    prefill = M.system_frames(tok, cfg, None)
    streamed = M.assistant_prefill(tok, cfg, M.ASSISTANT_OPEN, "hello there how are you fine thanks and you hello there", prefill)
    seen = []
    c1 = dec.backbone.new_cache()
    frames, stop = dec.generate_turn(c1, prefill, streamed, 6, 7, on_frame=lambda s, f: seen.append((s, list(f))))
    assert stop == "budget" and len(frames) == 6 and [s for s, _ in seen] == list(range(6)) and [f for _, f in seen] == frames
    assert all(len(f) == 4 and all(0 <= t < cfg.audio_vocab_size for t in f) for f in frames)
    assert c1.offset == len(prefill) + 5                                     # the last frame is never fed back
    assert dec.generate_turn(dec.backbone.new_cache(), prefill, streamed, 6, 7)[0] == frames
    assert dec.generate_turn(dec.backbone.new_cache(), prefill, streamed, 6, 8)[0] != frames
    assert dec.generate_turn(dec.backbone.new_cache(), prefill, streamed, 6, 7, cancel=lambda: True) is None
    assert dec.generate_turn(dec.backbone.new_cache(), prefill, streamed, 6, 7, on_frame=lambda s, f: False) is None
    # replaying the same frames leaves the cache where generating one more frame would find it
    c2 = dec.backbone.new_cache()
    assert dec.replay_turn(c2, prefill, streamed, frames) and c2.offset == len(prefill) + 6
    assert not dec.replay_turn(dec.backbone.new_cache(), prefill, streamed, frames, cancel=lambda: True)
    # an end token on codebook 0 stops the turn without emitting that frame
    monkeypatch.setattr(M, "min_eos_frames", lambda budget: 0)
    orig = dec.local.decode_frame
    calls = [0]

    def fake(hidden, history, p, rng, suppress):
        calls[0] += 1
        return [cfg.audio_eos, 0, 0, 0] if calls[0] == 3 else orig(hidden, history, p, rng, suppress)
    monkeypatch.setattr(dec.local, "decode_frame", fake)
    frames, stop = dec.generate_turn(dec.backbone.new_cache(), prefill, streamed, 6, 7)
    assert stop == "eos" and len(frames) == 2


def _restated_stage(w, p, x, context):
    h = x.transpose(1, 2)
    if p + "input_proj.weight" in w:
        h = h @ w[p + "input_proj.weight"].t()
    T, d = h.shape[1], h.shape[2]
    H, D = d // 64, 64
    inv = 10000.0 ** (-torch.arange(0, D, 2, dtype=torch.float64) / D)
    th = (torch.arange(T, dtype=torch.float64)[:, None] * inv).float()
    i = torch.arange(T)
    mask = torch.where((i[None, :] <= i[:, None]) & (i[:, None] - i[None, :] < context), 0.0, float("-inf"))

    def rope(v):                              # [1, H, T, D], adjacent pairs
        a, b = v[..., 0::2], v[..., 1::2]
        return torch.stack([a * th.cos() - b * th.sin(), a * th.sin() + b * th.cos()], -1).flatten(-2)

    li = 0
    while f"{p}transformer.layers.{li}.norm1.weight" in w:
        b = f"{p}transformer.layers.{li}."
        y = F.layer_norm(h, (d,), w[b + "norm1.weight"], w[b + "norm1.bias"], 1e-5)
        qkv = (y @ w[b + "self_attn.in_projs.0.weight"].t()).view(1, T, 3, H, D)
        q, k, v = (qkv[:, :, n].transpose(1, 2) for n in range(3))
        att = torch.softmax(rope(q) @ rope(k).transpose(-1, -2) / math.sqrt(D) + mask, -1) @ v
        h = h + (att.transpose(1, 2).reshape(1, T, d) @ w[b + "self_attn.out_projs.0.weight"].t()) * w[b + "layer_scale_1.scale"]
        y = F.layer_norm(h, (d,), w[b + "norm2.weight"], w[b + "norm2.bias"], 1e-5)
        h = h + (F.gelu(y @ w[b + "linear1.weight"].t()) @ w[b + "linear2.weight"].t()) * w[b + "layer_scale_2.scale"]
        li += 1
    if p + "output_proj.weight" in w:
        h = h @ w[p + "output_proj.weight"].t()
    return h.transpose(1, 2)


def test_codec_against_restatement_and_its_causality(snap):
    from inference_b200.contracts.errors import LoadError
    from inference_b200.io.safetensors_io import load_file

    codec = M.MossAudioCodec(snap[1], 4)
    assert (codec.hop, codec.sample_rate, codec.nq, len(codec.stages)) == (24, 24_000, 4, 4)
    assert [s.context for s in codec.stages] == [4, 8, 16, 32] and [s.heads for s in codec.stages] == [2, 2, 2, 2]
    raw = {k: v.float() for k, v in load_file(snap[1] / "model.safetensors").items()}
    x = torch.randn(1, 24, 9, generator=torch.Generator().manual_seed(0))
    got = codec.stages[0].forward(x)
    assert torch.allclose(got, _restated_stage(raw, "decoder.0.", x, 4), atol=2e-5)
    assert not torch.allclose(got, _restated_stage(raw, "decoder.0.", x, 64), atol=1e-4)     # the band is active at 9 frames
    m = M.band_mask(5, 2, "cpu")
    assert m.tolist() == [[j <= i and i - j < 2 for j in range(5)] for i in range(5)]
    # patching: channel groups become consecutive time steps, and back
    t = torch.arange(2 * 6 * 3, dtype=torch.float32).view(2, 6, 3)
    u = M.unpatch(t, 2)
    assert u.shape == (2, 3, 6) and u[0, 0].tolist() == [0, 3, 1, 4, 2, 5] and torch.equal(M.patch(u, 2), t)
    # decode: the explicit quantiser sum, and causality (a prefix of frames decodes to a prefix of the samples)
    g = torch.Generator().manual_seed(1)
    frames = torch.randint(0, 11, (14, 4), generator=g).tolist()
    pcm = codec.decode_frames(frames)
    assert pcm.shape == (14 * 24,) and torch.isfinite(pcm).all()
    fold = lambda p: M.fold_weight_norm_1x1(raw, p)                                        # noqa: E731
    emb = sum(raw[f"quantizer.quantizers.{q}.codebook.weight"][torch.tensor([min(f[q], 7) for f in frames])] @ fold(f"quantizer.quantizers.{q}.out_proj")[0].t()
              + fold(f"quantizer.quantizers.{q}.out_proj")[1] for q in range(4))
    y = (emb @ fold("quantizer.output_proj")[0].t() + fold("quantizer.output_proj")[1]).t()[None]
    for si, pz in enumerate((2, 2, 2, 3)):
        y = M.unpatch(_restated_stage(raw, f"decoder.{2 * si}.", y, codec.stages[si].context), pz)
    assert torch.allclose(pcm, y[0, 0], atol=5e-4)
    for k in (1, 5, 9):
        assert torch.allclose(codec.decode_frames(frames[:k]), pcm[: k * 24], atol=1e-4), k
    assert codec.decode_frames([]).numel() == 0 and codec.decode_frames(frames, cancel=lambda: True) is None
    # encode: floor(T / hop) frames of nq in-range codes; a foreign sample rate is resampled first
    wave = torch.randn(24 * 6 + 7, generator=g) * 0.3
    codes = codec.encode(wave, 24_000)
    assert len(codes) == 6 and all(len(c) == 4 and all(0 <= t < 8 for t in c) for c in codes)
    assert codec.encode(wave[:10], 24_000) == [] and len(codec.encode(wave, 48_000)) == 3
    assert torch.equal(M.resample_linear(wave, 24_000, 24_000), wave)
    up = M.resample_linear(torch.tensor([0.0, 1.0, 2.0]), 1, 2)
    assert up.tolist() == [0.0, 0.5, 1.0, 1.5, 2.0, 2.0]
    with pytest.raises(LoadError):
        M.MossAudioCodec(snap[1], 7)
    with pytest.raises(LoadError):
        M.MossAudioCodec(snap[1].parent, 4)


def test_streaming_chunker_with_a_fake_codec():
    class Fake:
        sample_rate, hop = 24_000, 10

        def __init__(self, cancel_after=None):
            self.cancel_after = cancel_after

        def decode_frames(self, frames, cancel=lambda: False):
            if cancel() or (self.cancel_after is not None and len(frames) > self.cancel_after):
                return None
            return torch.tensor([float(f[0]) for f in frames]).repeat_interleave(10)

    chunks = []
    ch = M.StreamingChunker(Fake(), 8, chunks.append)
    for i in range(20):
        assert ch.push([i + 1, 0, 0, 0])
        if i == 7:
            assert len(chunks) == 1                     # the first block is out long before the last frame exists
    pcm = ch.finish()
    assert [c.index for c in chunks] == [0, 1, 2] and [len(c.samples) for c in chunks] == [80, 80, 40]
    assert torch.equal(torch.tensor(sum((c.samples for c in chunks), [])), pcm) and pcm.numel() == 200
    assert torch.equal(pcm, Fake().decode_frames([[i + 1] for i in range(20)]))
    stopped = M.StreamingChunker(Fake(cancel_after=8), 8)
    assert all(stopped.push([1, 0, 0, 0]) for _ in range(15)) and not stopped.push([1, 0, 0, 0])
    assert M.frames_per_block(125) == 8 and M.frames_per_block(5) == 3 and M.frames_per_block(1) == 1


def test_generator_conformance_streaming_clone_and_conversations(snap, monkeypatch):
    from inference_b200.audio.catalog import provider_registry
    from inference_b200.contracts.errors import InferenceError, LoadError, Unsupported
    from inference_b200.contracts.gen_core import AudioTrack, ConversationTurn, GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import AudioParams, Conditioning, ConditioningKind
    from inference_b200.contracts.gen_core.runtime import ProgressStep, WeightsSource
    from inference_b200.testkit.audio_generator import AudioProfile, audio_conformance

    model, codec = snap
    reg = provider_registry("cpu")
    assert "cpu_moss_tts_realtime" in reg.ids()
    spec = LoadSpec.from_dir(model)
    spec.components["codec"] = WeightsSource.dir(codec)
    gen = reg.load("cpu_moss_tts_realtime", spec)
    d = gen.descriptor()
    caps = d.capabilities
    assert d.required_components == ["codec"] and caps.supports_streaming and caps.supports_conversation_history
    assert caps.supports_conversation_session and caps.audio_sample_rates == [24_000] and caps.max_audio_duration_secs == 2400.0
    monkeypatch.setattr(M, "DEFAULT_SECONDS", 0.8)                              # 10 frames
    monkeypatch.setattr(M, "min_eos_frames", lambda budget: budget)
    audio_conformance(gen, AudioProfile(prompt="hello there how are you"))
    # streaming: the chunks concatenate to the returned track, which equals the plain call's
    req = lambda **kw: GenerationRequest(prompt="hello there how are you fine thanks and you", seed=3,       # noqa: E731
                                         audio=AudioParams(target_duration=1.6), **kw)
    plain = gen.generate(req()).audio
    chunks, steps = [], []
    streamed = gen.generate_streaming(req(), lambda p: steps.append(p), chunks.append).audio
    assert streamed.samples == plain.samples and len(plain.samples) == 20 * 24
    assert [c.index for c in chunks] == [0, 1, 2] and sum((c.samples for c in chunks), []) == plain.samples
    assert [s.current for s in steps if isinstance(s, ProgressStep)] == list(range(1, 21))
    # voice clone: a reference clip changes the prompt and so the speech
    g = torch.Generator().manual_seed(5)
    clip = AudioTrack(24_000, 2, (torch.randn(2 * 24 * 5, generator=g) * 0.3).tolist())
    cloned = gen.generate(req(conditioning=[Conditioning(ConditioningKind.REFERENCE_AUDIO, audio=clip)])).audio
    assert len(cloned.samples) == len(plain.samples) and cloned.samples != plain.samples
    assert len(gen.reference_codes(req(conditioning=[Conditioning(ConditioningKind.REFERENCE_AUDIO, audio=clip)]))) == 5
    with pytest.raises(InferenceError):
        gen.generate(req(conditioning=[Conditioning(ConditioningKind.REFERENCE_AUDIO, audio=AudioTrack(24_000, 1, [0.0] * 10))]))
    # conversation: one request with the history == the same turns through a session
    user_audio = AudioTrack(24_000, 1, (torch.randn(24 * 4, generator=g) * 0.3).tolist())
    given = AudioTrack(24_000, 1, (torch.randn(24 * 3, generator=g) * 0.3).tolist())
    turns = [ConversationTurn("user", "hello there", user_audio), ConversationTurn("assistant", "fine thanks and you"),
             ConversationTurn("assistant", "how are you", given), ConversationTurn("user", "and you", user_audio),
             ConversationTurn("assistant", "hello there how are you")]
    creq = lambda: GenerationRequest(seed=11, audio=AudioParams(target_duration=0.4),                        # noqa: E731
                                     conditioning=[Conditioning(ConditioningKind.CONVERSATION_HISTORY, turns=turns)])
    psteps, cchunks = [], []
    batch = gen.generate_streaming(creq(), psteps.append, cchunks.append).audio
    assert len(batch.samples) == 2 * 5 * 24 and sum((c.samples for c in cchunks), []) == batch.samples
    assert [c.index for c in cchunks] == list(range(len(cchunks)))
    assert [s.current for s in psteps if isinstance(s, ProgressStep)] == list(range(1, 11))
    session = gen.open_conversation(GenerationRequest(seed=11, audio=AudioParams(target_duration=0.4)))
    out = [session.step(t) for t in turns]
    session.finish()
    assert out[0] is user_audio and out[2] is given                           # provided turns come back as given
    assert out[1].samples + out[4].samples == batch.samples
    assert out[1].samples != out[4].samples[: len(out[1].samples)]
    other = gen.open_conversation(GenerationRequest(seed=12, audio=AudioParams(target_duration=0.4)))
    assert other.step(turns[0]) is user_audio and other.step(turns[1]).samples != out[1].samples
    # request validation
    with pytest.raises(InferenceError):
        gen.validate(GenerationRequest(prompt=" "))
    for bad in ([], [ConversationTurn("user", "hi")], [ConversationTurn("narrator", "hi", user_audio)], [ConversationTurn("assistant", " ")]):
        with pytest.raises(InferenceError):
            gen.validate(GenerationRequest(conditioning=[Conditioning(ConditioningKind.CONVERSATION_HISTORY, turns=bad)]))
    with pytest.raises(InferenceError):
        session.step(ConversationTurn("user", "hello"))
    # load errors
    with pytest.raises(InferenceError):
        reg.load("cpu_moss_tts_realtime", LoadSpec.from_dir(model))
    bad = LoadSpec.from_dir(model)
    bad.components["codec"] = WeightsSource.file(codec / "model.safetensors")
    with pytest.raises(Unsupported):
        reg.load("cpu_moss_tts_realtime", bad)
    bad = LoadSpec.from_dir(model)
    bad.components.update(codec=WeightsSource.dir(codec), vocoder=WeightsSource.dir(codec))
    with pytest.raises(Unsupported):
        reg.load("cpu_moss_tts_realtime", bad)
    empty = LoadSpec.from_dir(codec)
    empty.components["codec"] = WeightsSource.dir(codec)
    with pytest.raises(LoadError):
        reg.load("cpu_moss_tts_realtime", empty).generate(GenerationRequest(prompt="hello"))
