"""Seconds per 1024x1024 image through the public generator API (`registry.load(model).generate(request)`):
prompt encoding, seeded CPU noise -> device, the flow-matching steps of the full-size DiT (FLUX.1-dev: 28 steps of
19 + 38 blocks; `--model chroma1_hd`: 28 steps, two forwards each; `--model z_image_turbo`: 4 steps of 30 + 4 blocks;
`--model z_image`: 50 steps, two forwards each), VAE decode, RGB8 image back on the host. Weights are random-init on
the device (a snapshot directory holding only `swb_config.json` with "random_init"), the prompt encoder is the
weight-free hash encoder with the model's caption width."""
import argparse
import json
import os
import sys
import tempfile
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", type=int, default=1024)
    ap.add_argument("--model", default="flux1_dev")
    ap.add_argument("--steps", type=int, default=0, help="0 = the model's default")
    ap.add_argument("--images", type=int, default=2)
    ap.add_argument("--frames", type=int, default=0, help="video models: frames per clip (0 = the model's default)")
    args = ap.parse_args()
    from inference_b200.bundles import runtime_b200
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec

    d = tempfile.mkdtemp()
    with open(os.path.join(d, "swb_config.json"), "w") as f:
        json.dump({"text": "hash", "random_init": 0}, f)
    gen = runtime_b200.catalog().media().load(args.model, LoadSpec.from_dir(d))
    extra = {"guidance": 3.5} if args.model == "flux1_dev" else {}
    if args.model in ("chroma1_hd", "chroma1_base", "z_image", "qwen_image", "sd3_5_large", "sd3_5_medium", "sdxl", "kolors",
                      "wan2_2_t2v_14b"):
        extra["negative_prompt"] = "blurry, low quality"
    if args.frames:
        extra["frames"] = args.frames
    events = []
    req = lambda seed: GenerationRequest(prompt="a photo of a fox", width=args.size, height=args.size,  # noqa: E731
                                         steps=args.steps or None, seed=seed, **extra)
    t0 = time.perf_counter()
    gen.generate(req(0), events.append)                 # loads, captures the CUDA graph
    torch.cuda.synchronize()
    first_s = time.perf_counter() - t0
    times = []
    for i in range(args.images):
        t0 = time.perf_counter()
        out = gen.generate(req(1 + i), lambda e: None)
        times.append(time.perf_counter() - t0)          # the image bytes are on the host when generate returns
        pictures = out.images or out.video_frames
        assert len(pictures[0].pixels) == args.size * args.size * 3
    print(json.dumps({"metric": f"{args.model}_seconds_per_image", "size": args.size,
                      "steps": args.steps or "model default",
                      "s_per_image": round(min(times), 3), "frames": len(pictures) if out.video_frames else None, "s_per_image_all": [round(t, 3) for t in times],
                      "first_image_s_including_load_and_capture": round(first_s, 2), "n_gpus": 1,
                      "data": "random-init weights, hash prompt encoder"}))


if __name__ == "__main__":
    main()
