"""OpenVoice V2 tone-colour voice conversion, `openvoice_v2` (parity: candle-audio-openvoice/src/converter.rs,
reference_encoder.rs, spectrogram.rs, pipeline.rs, model.rs).

The converter is a VITS-family flow model: a posterior encoder (gated dilated-convolution WaveNet over the 513-bin
linear spectrogram) samples a latent, four mean-only coupling layers (each followed by a channel flip) run forward
conditioned on the source speaker's tone colour and backward conditioned on the target's, and a HiFi-GAN decoder
(transposed-convolution upsampling by 8 * 8 * 2 * 2 = 256 with three residual stacks per scale) renders the waveform.
The tone colour is the final GRU state of a strided-convolution stack over a reference clip's spectrogram. The
checkpoint's `zero_g` setting feeds a zero vector to the posterior encoder and the decoder, so the whole timbre change
happens in the flow. Audio runs at 22.05 kHz (n_fft 1024, hop 256).

Checkpoint: the upstream `checkpoint.pth` state dict ("model" section) or the same tensors in safetensors; old-style
weight norm (`weight_g`, `weight_v`) is folded into plain weights at load."""
from __future__ import annotations

from pathlib import Path
from typing import Any

import torch
import torch.nn.functional as F

from ..contracts.errors import Canceled, InferenceError, LoadError
from ..contracts.gen_core.media import AudioTrack
from ..contracts.gen_core.traits import AudioTransform, SimpleDescriptor
from .clap import resample_linear
from .whisper import to_mono

MODEL_ID = "openvoice_v2"
SAMPLE_RATE, N_FFT, HOP = 22_050, 1024, 256
SPEC_BINS, INTER, HIDDEN, GIN = N_FFT // 2 + 1, 192, 192, 256
WN_KERNEL, ENC_LAYERS, FLOW_LAYERS, N_FLOWS = 5, 16, 4, 4
UP_RATES, UP_KERNELS, UP_INITIAL = (8, 8, 2, 2), (16, 16, 4, 4), 512
RES_KERNELS, RES_DILATIONS = (3, 7, 11), (1, 3, 5)
REF_FILTERS, REF_GRU = (32, 32, 64, 64, 128, 128), 128
DEFAULT_TAU = 0.3


def fold_weight_norm(sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """`x.weight_g`, `x.weight_v` -> `x.weight` = g * v / ||v|| (norm over every axis but the first); the newer
    parametrisation names (`parametrizations.weight.original0/1`) are folded the same way."""
    out = {}
    for k, v in sd.items():
        if k.endswith(("weight_g", "parametrizations.weight.original0")):
            continue
        if k.endswith("weight_v") or k.endswith("parametrizations.weight.original1"):
            base = k[: -len("weight_v")] if k.endswith("weight_v") else k[: -len("parametrizations.weight.original1")]
            g = sd.get(base + "weight_g", sd.get(base + "parametrizations.weight.original0"))
            norm = v.float().flatten(1).norm(dim=1).view(-1, *([1] * (v.dim() - 1)))
            out[base + "weight"] = (g.float().view_as(norm) * v.float() / norm).to(v.dtype)
        else:
            out[k] = v
    return out


def linear_spectrogram(wav: torch.Tensor) -> torch.Tensor:
    """[T] -> [513, frames]: reflect padding of (n_fft - hop) / 2 on both sides, un-centred Hann STFT,
    sqrt(re^2 + im^2 + 1e-6)."""
    pad = (N_FFT - HOP) // 2
    y = F.pad(wav.float()[None, None], (pad, pad), mode="reflect")[0, 0]
    spec = torch.stft(y, N_FFT, HOP, N_FFT, window=torch.hann_window(N_FFT, device=wav.device), center=False,
                      return_complex=True)
    return torch.sqrt(spec.real ** 2 + spec.imag ** 2 + 1e-6)


def gru_last_state(x: torch.Tensor, w_ih, w_hh, b_ih, b_hh) -> torch.Tensor:
    """x [T, in] -> final hidden state [hidden] (gate order r, z, n)."""
    H = w_hh.shape[1]
    h = torch.zeros(H, dtype=x.dtype, device=x.device)
    gi = x @ w_ih.t() + b_ih
    for t in range(x.shape[0]):
        gh = w_hh @ h + b_hh
        r = torch.sigmoid(gi[t, :H] + gh[:H])
        z = torch.sigmoid(gi[t, H:2 * H] + gh[H:2 * H])
        n = torch.tanh(gi[t, 2 * H:] + r * gh[2 * H:])
        h = (1 - z) * n + z * h
    return h


class OpenVoiceConverter:
    def __init__(self, weights: dict[str, torch.Tensor], device="cpu", dtype=torch.float32):
        self.device, self.dtype = torch.device(device), dtype
        self.w = {k: v.to(device=self.device, dtype=dtype).contiguous() for k, v in fold_weight_norm(weights).items()}
        for need in ("enc_q.pre.weight", "flow.flows.0.pre.weight", "dec.conv_pre.weight", "ref_enc.proj.weight"):
            if need not in self.w:
                raise LoadError(f"{MODEL_ID}: checkpoint lacks {need}")

    def _c1(self, x, name, **kw):
        return F.conv1d(x, self.w[name + ".weight"], self.w.get(name + ".bias"), **kw)

    # ---- tone colour ---------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def tone_color(self, spec: torch.Tensor) -> torch.Tensor:
        """spectrogram [513, frames] -> g [1, 256, 1]."""
        w = self.w
        x = spec.t().to(self.device, self.dtype)                                        # [frames, 513]
        if "ref_enc.layernorm.weight" in w:
            x = F.layer_norm(x, (SPEC_BINS,), w["ref_enc.layernorm.weight"], w["ref_enc.layernorm.bias"])
        x = x[None, None]
        for i in range(len(REF_FILTERS)):
            x = F.relu(F.conv2d(x, w[f"ref_enc.convs.{i}.weight"], w[f"ref_enc.convs.{i}.bias"], stride=2, padding=1))
        x = x[0].permute(1, 0, 2).reshape(x.shape[2], -1)                               # [frames', 128 * bins']
        h = gru_last_state(x, w["ref_enc.gru.weight_ih_l0"], w["ref_enc.gru.weight_hh_l0"], w["ref_enc.gru.bias_ih_l0"],
                           w["ref_enc.gru.bias_hh_l0"])
        return (w["ref_enc.proj.weight"] @ h + w["ref_enc.proj.bias"]).view(1, GIN, 1)

    # ---- shared WaveNet ------------------------------------------------------------------------------------------------------
    def _wavenet(self, x, g, p, layers):
        out = torch.zeros_like(x)
        cond = self._c1(g, p + ".cond_layer") if g is not None and p + ".cond_layer.weight" in self.w else None
        for i in range(layers):
            a = self._c1(x, f"{p}.in_layers.{i}", padding=(WN_KERNEL - 1) // 2)
            if cond is not None:
                a = a + cond[:, 2 * HIDDEN * i: 2 * HIDDEN * (i + 1)]
            a = torch.tanh(a[:, :HIDDEN]) * torch.sigmoid(a[:, HIDDEN:])
            rs = self._c1(a, f"{p}.res_skip_layers.{i}")
            if i < layers - 1:
                x = x + rs[:, :HIDDEN]
                out = out + rs[:, HIDDEN:]
            else:
                out = out + rs
        return out

    def posterior(self, spec, g, tau, noise):
        """[1, 513, T] -> latent [1, 192, T] = mean + noise * tau * exp(log-scale)."""
        h = self._wavenet(self._c1(spec, "enc_q.pre"), g, "enc_q.enc", ENC_LAYERS)
        m, logs = self._c1(h, "enc_q.proj").chunk(2, 1)
        return m + noise * tau * torch.exp(logs)

    def _coupling_mean(self, x0, g, i):
        p = f"flow.flows.{2 * i}"
        return self._c1(self._wavenet(self._c1(x0, p + ".pre"), g, p + ".enc", FLOW_LAYERS), p + ".post")

    def flow(self, z, g, reverse: bool):
        half = INTER // 2
        order = range(N_FLOWS - 1, -1, -1) if reverse else range(N_FLOWS)
        for i in order:
            if reverse:
                z = z.flip(1)                                   # undo the flip that followed this coupling layer
                x0, x1 = z[:, :half], z[:, half:]
                z = torch.cat([x0, x1 - self._coupling_mean(x0, g, i)], 1)
            else:
                x0, x1 = z[:, :half], z[:, half:]
                z = torch.cat([x0, x1 + self._coupling_mean(x0, g, i)], 1).flip(1)
        return z

    def decode(self, z, g):
        x = self._c1(z, "dec.conv_pre", padding=3)
        if g is not None and "dec.cond.weight" in self.w:
            x = x + self._c1(g, "dec.cond")
        nk = len(RES_KERNELS)
        for i, (u, k) in enumerate(zip(UP_RATES, UP_KERNELS)):
            x = F.conv_transpose1d(F.leaky_relu(x, 0.1), self.w[f"dec.ups.{i}.weight"], self.w[f"dec.ups.{i}.bias"],
                                   stride=u, padding=(k - u) // 2)
            acc = None
            for j, rk in enumerate(RES_KERNELS):
                p = f"dec.resblocks.{i * nk + j}"
                y = x
                for d_i, d in enumerate(RES_DILATIONS):
                    t = self._c1(F.leaky_relu(y, 0.1), f"{p}.convs1.{d_i}", dilation=d, padding=d * (rk - 1) // 2)
                    y = y + self._c1(F.leaky_relu(t, 0.1), f"{p}.convs2.{d_i}", padding=(rk - 1) // 2)
                acc = y if acc is None else acc + y
            x = acc / nk
        return torch.tanh(self._c1(F.leaky_relu(x), "dec.conv_post", padding=3))

    @torch.no_grad()
    def convert(self, spec: torch.Tensor, g_src: torch.Tensor, g_tgt: torch.Tensor, tau: float, noise: torch.Tensor,
                cancelled=lambda: False) -> torch.Tensor:
        """spectrogram [513, T] -> waveform [T * 256] in the target's tone colour."""
        s = spec.to(self.device, self.dtype)[None]
        zero = torch.zeros(1, GIN, 1, device=self.device, dtype=self.dtype)       # the checkpoint's zero_g setting
        z = self.posterior(s, zero, tau, noise.to(self.device, self.dtype))
        for step in (lambda v: self.flow(v, g_src, False), lambda v: self.flow(v, g_tgt, True)):
            if cancelled():
                raise Canceled(f"{MODEL_ID}: cancelled")
            z = step(z)
        if cancelled():
            raise Canceled(f"{MODEL_ID}: cancelled")
        return self.decode(z, zero)[0, 0]


def _mono_22k(track: AudioTrack) -> torch.Tensor:
    return resample_linear(to_mono(torch.tensor(track.samples, dtype=torch.float32), track.channels), track.sample_rate,
                           SAMPLE_RATE)


class OpenVoiceTransform(AudioTransform):
    """apply(audio, params): params["target_reference"] is the AudioTrack whose voice the output should have; optional
    "tau" (default 0.3) scales the sampled latent noise, "seed" fixes it, "cancel" is a cancellation flag."""

    def __init__(self, converter: OpenVoiceConverter, backend: str):
        self.model, self.backend = converter, backend

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor(MODEL_ID, "openvoice", self.backend, {"sample_rate": SAMPLE_RATE, "needs": ["target_reference"]})

    def apply(self, audio: AudioTrack, params: dict[str, Any] | None = None) -> AudioTrack:
        params = params or {}
        ref = params.get("target_reference")
        if not isinstance(ref, AudioTrack):
            raise InferenceError(f"{MODEL_ID}: params['target_reference'] must be the target voice's AudioTrack")
        src, tgt = _mono_22k(audio), _mono_22k(ref)
        for name, wav in (("audio", src), ("target_reference", tgt)):
            if wav.numel() < N_FFT:
                raise InferenceError(f"{MODEL_ID}: {name} is shorter than {N_FFT} samples at {SAMPLE_RATE} Hz")
        cancel = params.get("cancel")
        spec = linear_spectrogram(src)
        g_src = self.model.tone_color(spec)
        g_tgt = self.model.tone_color(linear_spectrogram(tgt))
        gen = torch.Generator().manual_seed(int(params.get("seed", 0)))
        noise = torch.randn(1, INTER, spec.shape[1], generator=gen)
        out = self.model.convert(spec, g_src, g_tgt, float(params.get("tau", DEFAULT_TAU)), noise,
                                 (lambda: cancel.is_cancelled()) if cancel is not None else (lambda: False))
        return AudioTrack(SAMPLE_RATE, 1, out.float().cpu().tolist())


def load_checkpoint(path: str | Path) -> dict[str, torch.Tensor]:
    """A directory holding `checkpoint.pth` / `*.safetensors`, or such a file."""
    p = Path(path)
    if p.is_dir():
        cands = sorted(p.glob("*.safetensors")) + sorted(p.glob("checkpoint*.pth"))
        if not cands:
            raise LoadError(f"{MODEL_ID}: {p} holds neither *.safetensors nor checkpoint.pth")
        p = cands[0]
    if p.suffix == ".safetensors":
        from ..io.safetensors_io import load_file

        return load_file(p)
    sd = torch.load(p, map_location="cpu", weights_only=True)
    return sd.get("model", sd)


def random_openvoice_weights(seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    """A random checkpoint with the real tensor names and shapes (old-style weight norm on the reference encoder's
    convolutions, as upstream stores it)."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g) * std      # noqa: E731
    w: dict[str, torch.Tensor] = {}

    def conv(name, o, i, k, bias=True):
        w[name + ".weight"] = rn(o, i, k)
        if bias:
            w[name + ".bias"] = rn(o)

    def wavenet(p, layers, gin):
        if gin:
            conv(p + ".cond_layer", 2 * HIDDEN * layers, gin, 1)
        for i in range(layers):
            conv(f"{p}.in_layers.{i}", 2 * HIDDEN, HIDDEN, WN_KERNEL)
            conv(f"{p}.res_skip_layers.{i}", 2 * HIDDEN if i < layers - 1 else HIDDEN, HIDDEN, 1)

    conv("enc_q.pre", HIDDEN, SPEC_BINS, 1)
    wavenet("enc_q.enc", ENC_LAYERS, GIN)
    conv("enc_q.proj", 2 * INTER, HIDDEN, 1)
    for i in range(N_FLOWS):
        p = f"flow.flows.{2 * i}"
        conv(p + ".pre", HIDDEN, INTER // 2, 1)
        wavenet(p + ".enc", FLOW_LAYERS, GIN)
        conv(p + ".post", INTER // 2, HIDDEN, 1)
    conv("dec.conv_pre", UP_INITIAL, INTER, 7)
    conv("dec.cond", UP_INITIAL, GIN, 1)
    ch = UP_INITIAL
    for i, (u, k) in enumerate(zip(UP_RATES, UP_KERNELS)):
        w[f"dec.ups.{i}.weight"], w[f"dec.ups.{i}.bias"] = rn(ch, ch // 2, k), rn(ch // 2)
        ch //= 2
        for j, rk in enumerate(RES_KERNELS):
            for d in range(len(RES_DILATIONS)):
                conv(f"dec.resblocks.{i * len(RES_KERNELS) + j}.convs1.{d}", ch, ch, rk)
                conv(f"dec.resblocks.{i * len(RES_KERNELS) + j}.convs2.{d}", ch, ch, rk)
    conv("dec.conv_post", 1, ch, 7, bias=False)
    cin = 1
    for i, f in enumerate(REF_FILTERS):
        v = torch.randn(f, cin, 3, 3, generator=g) * 0.3
        w[f"ref_enc.convs.{i}.weight_v"] = v
        w[f"ref_enc.convs.{i}.weight_g"] = v.flatten(1).norm(dim=1).view(-1, 1, 1, 1) * 1.1
        w[f"ref_enc.convs.{i}.bias"] = rn(f)
        cin = f
    bins = SPEC_BINS
    for _ in REF_FILTERS:
        bins = (bins - 3 + 2) // 2 + 1
    w["ref_enc.layernorm.weight"], w["ref_enc.layernorm.bias"] = 1.0 + rn(SPEC_BINS), rn(SPEC_BINS)
    w["ref_enc.gru.weight_ih_l0"], w["ref_enc.gru.weight_hh_l0"] = rn(3 * REF_GRU, REF_FILTERS[-1] * bins), rn(3 * REF_GRU, REF_GRU)
    w["ref_enc.gru.bias_ih_l0"], w["ref_enc.gru.bias_hh_l0"] = rn(3 * REF_GRU), rn(3 * REF_GRU)
    w["ref_enc.proj.weight"], w["ref_enc.proj.bias"] = rn(GIN, REF_GRU), rn(GIN)
    return w
