"""Seconds per 1024x1024 image through the public generator API (`registry.load("flux1_dev").generate(request)`):
prompt encoding, seeded CPU noise -> device, 28 flow-matching steps of the full 19 + 38 block DiT, VAE decode, RGB8
image back on the host. Weights are random-init on the device (a snapshot directory holding only
`swb_config.json` with "random_init"), the prompt encoder is the weight-free hash encoder with FLUX's shapes."""
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
    ap.add_argument("--steps", type=int, default=28)
    ap.add_argument("--images", type=int, default=2)
    args = ap.parse_args()
    from inference_b200.bundles import runtime_b200
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec

    d = tempfile.mkdtemp()
    with open(os.path.join(d, "swb_config.json"), "w") as f:
        json.dump({"text": "hash", "random_init": 0}, f)
    gen = runtime_b200.catalog().media().load("flux1_dev", LoadSpec.from_dir(d))
    events = []
    req = lambda seed: GenerationRequest(prompt="a photo of a fox", width=args.size, height=args.size,  # noqa: E731
                                         steps=args.steps, seed=seed, guidance=3.5)
    t0 = time.perf_counter()
    gen.generate(req(0), events.append)                 # loads, captures the CUDA graph
    torch.cuda.synchronize()
    first_s = time.perf_counter() - t0
    times = []
    for i in range(args.images):
        t0 = time.perf_counter()
        out = gen.generate(req(1 + i), lambda e: None)
        times.append(time.perf_counter() - t0)          # the image bytes are on the host when generate returns
        assert len(out.images[0].pixels) == args.size * args.size * 3
    print(json.dumps({"metric": "flux1_dev_seconds_per_image", "size": args.size, "steps": args.steps,
                      "s_per_image": round(min(times), 3), "s_per_image_all": [round(t, 3) for t in times],
                      "first_image_s_including_load_and_capture": round(first_s, 2), "n_gpus": 1,
                      "data": "random-init weights, hash prompt encoder"}))


if __name__ == "__main__":
    main()
