"""FLUX IP-Adapter: token projection and per-block residual against explicit math, the image-query seam of the base model
(scale 0 is the base model bit for bit; composition with another injector), and the bespoke provider end to end."""
import json
import math

import pytest
import torch
import torch.nn.functional as F

from inference_b200.media import flux_ip as P
from inference_b200.models.dit_flux import FluxConfig, OracleFluxDiT, make_ids, random_flux_weights


def test_adapter_tokens_and_block_residual():
    from inference_b200.contracts.errors import LoadError

    w = P.random_ip_adapter_weights(blocks=2, hidden=256, embed_dim=24, cross_dim=32, seed=1)
    ad = P.FluxIpAdapter(w)
    assert (ad.blocks, ad.num_tokens, ad.cross_dim) == (2, 4, 32)
    emb = torch.randn(1, 24, generator=torch.Generator().manual_seed(2))
    tok = ad.tokens(emb)
    want = F.layer_norm(F.linear(emb, w["ip_adapter_proj_model.proj.weight"], w["ip_adapter_proj_model.proj.bias"]).view(1, 4, 32), (32,),
                        w["ip_adapter_proj_model.norm.weight"], w["ip_adapter_proj_model.norm.bias"], 1e-5)
    assert tok.shape == (1, 4, 32) and torch.allclose(tok, want, atol=1e-6)
    q = torch.randn(1, 6, 2, 128, generator=torch.Generator().manual_seed(3))
    inj = P.FluxIpInjector(ad, tok, 0.7)
    inj.on_img_query(1, q)
    r = inj.after_double(1, None)
    p = "double_blocks.1.processor.ip_adapter_double_stream_"
    k = F.linear(tok, w[p + "k_proj.weight"], w[p + "k_proj.bias"]).view(1, 4, 2, 128).transpose(1, 2)
    v = F.linear(tok, w[p + "v_proj.weight"], w[p + "v_proj.bias"]).view(1, 4, 2, 128).transpose(1, 2)
    ref = (torch.softmax(q.transpose(1, 2) @ k.transpose(-1, -2) / math.sqrt(128), -1) @ v).transpose(1, 2).reshape(1, 6, 256) * 0.7
    assert torch.allclose(r, ref, atol=1e-5)
    assert inj.after_double(1, None) is None                      # the query is consumed; nothing stale leaks into a later call
    kv = inj.kv[1]
    inj.on_img_query(1, q)
    inj.after_double(1, None)
    assert inj.kv[1][0] is kv[0]                                 # keys / values are computed once per generation
    inj.on_img_query(5, q)
    assert inj.after_double(5, None) is None                     # blocks beyond the adapter's pairs are untouched
    off = P.FluxIpInjector(ad, tok, 0.0)
    off.on_img_query(0, q)
    assert off.after_double(0, None) is None
    with pytest.raises(LoadError):
        P.FluxIpAdapter({k_: v_ for k_, v_ in w.items() if not k_.startswith("double_blocks.")})
    with pytest.raises(LoadError):
        P.FluxIpAdapter({k_: v_ for k_, v_ in w.items() if k_ != "ip_adapter_proj_model.norm.bias"})


def test_seam_in_the_base_model():
    cfg = FluxConfig.tiny()
    base = OracleFluxDiT(cfg, random_flux_weights(cfg, 2, std=0.05))
    g = torch.Generator().manual_seed(0)
    img, txt = torch.randn(1, 6, cfg.in_channels, generator=g), torch.randn(1, 5, cfg.context_in_dim, generator=g)
    y = torch.randn(1, cfg.vec_in_dim, generator=g)
    txt_ids, img_ids = make_ids(2, 3, 5)
    t, gd = torch.tensor([0.6]), torch.tensor([3.5])
    plain = base.forward(img, img_ids, txt, txt_ids, t, y, gd)
    ad = P.FluxIpAdapter(P.random_ip_adapter_weights(cfg.depth, cfg.hidden_size, 24, seed=4))
    tok = ad.tokens(torch.randn(1, 24, generator=g))
    seen = []

    class Spy(P.FluxIpInjector):
        def on_img_query(self, i, q):
            seen.append((i, tuple(q.shape)))
            super().on_img_query(i, q)
    base.injector = Spy(ad, tok, 0.7)
    out = base.forward(img, img_ids, txt, txt_ids, t, y, gd)
    assert seen == [(i, (1, 6, cfg.num_heads, cfg.head_dim)) for i in range(cfg.depth)]
    assert not torch.allclose(out, plain, atol=1e-4)
    base.injector = P.FluxIpInjector(ad, tok, 0.0)
    assert torch.equal(base.forward(img, img_ids, txt, txt_ids, t, y, gd), plain)

    class Inner:
        def after_double(self, i, im):             # not constant over channels: the layer norms would erase that
            return 0.3 * torch.sin(torch.arange(im.shape[-1], dtype=im.dtype)).expand_as(im)

        def after_single(self, i, im):
            return -0.3 * torch.cos(torch.arange(im.shape[-1], dtype=im.dtype)).expand_as(im)
    base.injector = Inner()
    only_inner = base.forward(img, img_ids, txt, txt_ids, t, y, gd)
    base.injector = P.FluxIpInjector(ad, tok, 0.0, Inner())
    assert torch.equal(base.forward(img, img_ids, txt, txt_ids, t, y, gd), only_inner)
    base.injector = P.FluxIpInjector(ad, tok, 0.7, Inner())
    both = base.forward(img, img_ids, txt, txt_ids, t, y, gd)
    assert not torch.allclose(both, only_inner, atol=1e-4) and not torch.allclose(both, out, atol=1e-4)
    base.injector = None


def _write_clip(d):
    from transformers import CLIPConfig, CLIPModel

    from inference_b200.io.safetensors_io import save_file

    torch.manual_seed(3)
    hc = CLIPConfig(text_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4, vocab_size=100,
                                     max_position_embeddings=8),
                    vision_config=dict(hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, image_size=28,
                                       patch_size=14), projection_dim=24)
    d.mkdir()
    (d / "config.json").write_text(json.dumps(hc.to_dict()))
    save_file({k: v.contiguous() for k, v in CLIPModel(hc).eval().state_dict().items()}, d / "model.safetensors")


def test_provider_end_to_end(tmp_path):
    pytest.importorskip("transformers")
    from inference_b200.contracts.errors import Canceled, InferenceError, LoadError
    from inference_b200.contracts.gen_core import GenerationRequest
    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.io.safetensors_io import save_file
    from inference_b200.media import flux

    snap = flux.write_synthetic_snapshot(tmp_path / "flux", flux.Variant.SCHNELL)
    assert P.detect_variant(snap) == "flux1_schnell"
    with pytest.raises(LoadError):
        P.detect_variant(tmp_path)
    _write_clip(tmp_path / "clip")
    from inference_b200.contracts.gen_core.runtime import LoadSpec
    from inference_b200.media.catalog import provider_registry
    cfg = provider_registry("cpu").load("cpu_flux1_schnell", LoadSpec.from_dir(snap)).pipe.dit_cfg
    save_file(P.random_ip_adapter_weights(cfg.depth, cfg.hidden_size, 24, seed=5), tmp_path / "ip_adapter.safetensors")
    save_file(P.random_ip_adapter_weights(cfg.depth + 1, cfg.hidden_size, 24, seed=5), tmp_path / "too_many.safetensors")
    paths = P.IpAdapterFluxPaths(snap, tmp_path / "ip_adapter.safetensors", tmp_path / "clip")
    with pytest.raises(LoadError):
        P.IpAdapterFlux.load(P.IpAdapterFluxPaths(snap, tmp_path / "missing.safetensors", tmp_path / "clip"), "cpu")
    with pytest.raises(LoadError):
        P.IpAdapterFlux.load(P.IpAdapterFluxPaths(snap, tmp_path / "too_many.safetensors", tmp_path / "clip"), "cpu")
    prov = P.IpAdapterFlux.load(paths, "cpu")
    g = torch.Generator().manual_seed(0)
    ref = Image(40, 30, bytes(torch.randint(0, 256, (30 * 40 * 3,), generator=g, dtype=torch.uint8).tolist()))
    emb = prov.image_embeds(ref)
    assert emb.shape == (1, 24) and abs(float(emb.norm()) - 1.0) > 1e-3            # the raw projection, not a unit vector
    req = lambda **kw: P.IpAdapterFluxRequest(**{**dict(prompt="a portrait in oil", width=256, height=256, steps=2, seed=5), **kw})   # noqa: E731
    img = prov.generate(req(), ref)
    assert (img.width, img.height) == (256, 256) and prov.generate(req(), ref).pixels == img.pixels
    plain = prov.flux.generate(GenerationRequest(prompt="a portrait in oil", width=256, height=256, steps=2, seed=5)).images[0]
    assert prov.generate(req(ip_adapter_scale=0.0), ref).pixels == plain.pixels and img.pixels != plain.pixels
    other = Image(40, 30, bytes(torch.randint(0, 256, (30 * 40 * 3,), generator=g, dtype=torch.uint8).tolist()))
    assert prov.generate(req(), other).pixels != img.pixels
    for bad in (dict(prompt=" "), dict(width=250), dict(steps=0), dict(ip_adapter_scale=float("inf"))):
        with pytest.raises(InferenceError):
            prov.generate(req(**bad), ref)
    done = req()
    done.cancel.cancel()
    with pytest.raises(Canceled):
        prov.generate(done, ref)
