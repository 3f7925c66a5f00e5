"""python -m inference_b200.server --model DIR_OR_GGUF [--host H] [--port P] [--provider ID] [--quant q4|q8]
[--bundle b200|cpu] [--no-batching] (role of mlx-llm-server's main.rs:68-165)."""
from __future__ import annotations

import argparse
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="inference_b200.server")
    ap.add_argument("--model", required=True, help="snapshot directory or GGUF file")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--provider", default=None, help="registry id (default: pick by model)")
    ap.add_argument("--quant", choices=["q4", "q8"], default=None)
    ap.add_argument("--bundle", choices=["b200", "cpu"], default="b200")
    ap.add_argument("--no-batching", action="store_true")
    ap.add_argument("--max-batch", type=int, default=64)
    args = ap.parse_args(argv)
    from ..bundles import runtime_b200, runtime_cpu
    from ..contracts.core_llm import LoadSpec, Quantize
    from .http import serve

    catalog = (runtime_b200 if args.bundle == "b200" else runtime_cpu).catalog()
    spec = LoadSpec(args.model, {"q4": Quantize.Q4, "q8": Quantize.Q8, None: None}[args.quant])
    reg = catalog.text()
    llm = reg.load_textllm(args.provider, spec) if args.provider else reg.load_for_model(spec)
    httpd, service = serve(llm, llm.descriptor().id, args.host, args.port, not args.no_batching, args.max_batch)
    try:
        httpd.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        httpd.server_close()
        service.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
