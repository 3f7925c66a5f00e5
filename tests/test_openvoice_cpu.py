"""OpenVoice V2 converter: posterior encoder, coupling flow and HiFi-GAN decoder against the Hugging Face VITS modules
carrying the same weights; the tone-colour encoder against torch.nn modules; the spectrogram front end; the provider."""
import pytest
import torch
import torch.nn as nn

from inference_b200.audio import openvoice as OV

vits = pytest.importorskip("transformers.models.vits.modeling_vits")


def _cfg():
    from transformers import VitsConfig

    return VitsConfig(hidden_size=192, flow_size=192, spectrogram_bins=513, speaker_embedding_size=256, wavenet_kernel_size=5,
                      wavenet_dilation_rate=1, posterior_encoder_num_wavenet_layers=16, prior_encoder_num_flows=4,
                      prior_encoder_num_wavenet_layers=4, upsample_initial_channel=512, upsample_rates=[8, 8, 2, 2],
                      upsample_kernel_sizes=[16, 16, 4, 4], resblock_kernel_sizes=[3, 7, 11],
                      resblock_dilation_sizes=[[1, 3, 5]] * 3, leaky_relu_slope=0.1)


def _set(conv, w, name):
    W = w[name + ".weight"]
    if hasattr(conv, "parametrizations"):          # weight-normed: v = W and g = ||W|| reproduce W
        conv.parametrizations.weight.original1.data.copy_(W)
        conv.parametrizations.weight.original0.data.copy_(W.flatten(1).norm(dim=1).view(-1, *([1] * (W.dim() - 1))))
    else:
        conv.weight.data.copy_(W)
    if conv.bias is not None:
        conv.bias.data.copy_(w[name + ".bias"])


def _fill_wavenet(wn, w, p, layers):
    _set(wn.cond_layer, w, p + ".cond_layer")
    for i in range(layers):
        _set(wn.in_layers[i], w, f"{p}.in_layers.{i}")
        _set(wn.res_skip_layers[i], w, f"{p}.res_skip_layers.{i}")


@pytest.fixture(scope="module")
def model():
    w = OV.random_openvoice_weights(seed=1, std=0.05)
    return w, OV.OpenVoiceConverter(w)


def test_posterior_flow_and_decoder_match_hugging_face_vits(model):
    w, conv = model
    cfg = _cfg()
    g = torch.Generator().manual_seed(0)
    T = 24
    spec, gvec = torch.rand(1, 513, T, generator=g), torch.randn(1, 256, 1, generator=g)
    mask = torch.ones(1, 1, T)
    pe = vits.VitsPosteriorEncoder(cfg).eval()
    _set(pe.conv_pre, w, "enc_q.pre")
    _set(pe.conv_proj, w, "enc_q.proj")
    _fill_wavenet(pe.wavenet, w, "enc_q.enc", 16)
    with torch.no_grad():
        _, mean, logstd = pe(spec, mask, gvec)
    torch.testing.assert_close(conv.posterior(spec, gvec, 0.0, torch.zeros(1, 192, T)), mean, atol=1e-5, rtol=1e-4)
    one = conv.posterior(spec, gvec, 1.0, torch.ones(1, 192, T))
    torch.testing.assert_close(one - mean, torch.exp(logstd), atol=1e-5, rtol=1e-4)
    fl = vits.VitsResidualCouplingBlock(cfg).eval()
    for i, layer in enumerate(fl.flows):
        p = f"flow.flows.{2 * i}"
        _set(layer.conv_pre, w, p + ".pre")
        _set(layer.conv_post, w, p + ".post")
        _fill_wavenet(layer.wavenet, w, p + ".enc", 4)
    z = torch.randn(1, 192, T, generator=g)
    with torch.no_grad():
        fwd, rev = fl(z, mask, gvec), fl(z, mask, gvec, reverse=True)
    torch.testing.assert_close(conv.flow(z, gvec, False), fwd, atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(conv.flow(z, gvec, True), rev, atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(conv.flow(conv.flow(z, gvec, False), gvec, True), z, atol=1e-5, rtol=1e-4)
    dec = vits.VitsHifiGan(cfg).eval()
    _set(dec.conv_pre, w, "dec.conv_pre")
    _set(dec.conv_post, w, "dec.conv_post")
    _set(dec.cond, w, "dec.cond")
    for i, up in enumerate(dec.upsampler):
        _set(up, w, f"dec.ups.{i}")
    for n, rb in enumerate(dec.resblocks):
        for d in range(3):
            _set(rb.convs1[d], w, f"dec.resblocks.{n}.convs1.{d}")
            _set(rb.convs2[d], w, f"dec.resblocks.{n}.convs2.{d}")
    with torch.no_grad():
        ref = dec(z, gvec)
    out = conv.decode(z, gvec)
    assert out.shape == (1, 1, T * 256)
    torch.testing.assert_close(out, ref, atol=1e-5, rtol=1e-4)


def test_tone_colour_encoder_matches_torch_modules(model):
    w, conv = model
    folded = OV.fold_weight_norm(w)
    spec = torch.rand(513, 140, generator=torch.Generator().manual_seed(2))
    x = nn.functional.layer_norm(spec.t(), (513,), folded["ref_enc.layernorm.weight"], folded["ref_enc.layernorm.bias"])[None, None]
    cin = 1
    for i, f in enumerate(OV.REF_FILTERS):
        c = nn.utils.weight_norm(nn.Conv2d(cin, f, 3, 2, 1))
        c.weight_g.data.copy_(w[f"ref_enc.convs.{i}.weight_g"])
        c.weight_v.data.copy_(w[f"ref_enc.convs.{i}.weight_v"])
        c.bias.data.copy_(w[f"ref_enc.convs.{i}.bias"])
        with torch.no_grad():
            x = torch.relu(c(x))
        cin = f
    x = x.transpose(1, 2).reshape(1, x.shape[2], -1)
    gru = nn.GRU(x.shape[-1], 128, batch_first=True)
    gru.load_state_dict({k[len("ref_enc.gru."):]: v for k, v in w.items() if k.startswith("ref_enc.gru.")})
    with torch.no_grad():
        ref = nn.functional.linear(gru(x)[1][0], w["ref_enc.proj.weight"], w["ref_enc.proj.bias"])
    torch.testing.assert_close(conv.tone_color(spec)[:, :, 0], ref, atol=1e-5, rtol=1e-4)


def test_spectrogram_front_end():
    wav = torch.sin(torch.arange(22_050) * 2 * torch.pi * 440 / 22_050)
    s = OV.linear_spectrogram(wav)
    assert s.shape == (513, 22_050 // 256) and s.min() >= 1e-3 - 1e-6            # sqrt(1e-6) floor
    assert int(s.mean(1).argmax()) == round(440 * 1024 / 22_050)


def test_provider_through_the_audio_catalog(tmp_path):
    from inference_b200.audio.catalog import provider_registry, weight_licenses
    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import LoadSpec
    from inference_b200.contracts.gen_core.media import AudioTrack
    from inference_b200.io.safetensors_io import save_file

    save_file(OV.random_openvoice_weights(seed=3), tmp_path / "converter.safetensors")
    reg = provider_registry("cpu")
    tr = reg.load_kind("audio_transform", "openvoice_v2", LoadSpec.from_dir(tmp_path))
    assert tr.descriptor().id == "openvoice_v2" and any(e.provider_id == "openvoice_v2" for e in weight_licenses())
    t = torch.arange(8000) / 16_000
    src = AudioTrack(16_000, 1, (0.3 * torch.sin(2 * torch.pi * 220 * t)).tolist())
    ref = AudioTrack(22_050, 2, (0.2 * torch.sin(2 * torch.pi * 330 * torch.arange(2 * 9000) / 44_100)).tolist())
    out = tr.apply(src, {"target_reference": ref, "seed": 7})
    frames = (8000 * 22_050 // 16_000) // 256
    assert out.sample_rate == 22_050 and out.channels == 1 and abs(len(out.samples) - frames * 256) <= 256
    assert max(abs(v) for v in out.samples) <= 1.0
    assert tr.apply(src, {"target_reference": ref, "seed": 7}).samples == out.samples
    assert tr.apply(src, {"target_reference": ref, "seed": 8}).samples != out.samples
    with pytest.raises(InferenceError):
        tr.apply(src, {})
    with pytest.raises(InferenceError):
        tr.apply(AudioTrack(22_050, 1, [0.0] * 100), {"target_reference": ref})
