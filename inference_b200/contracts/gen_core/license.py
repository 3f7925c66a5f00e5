"""Machine-readable model-weight licenses (gen-core/src/license.rs:34-120): each provider declares the license of the
checkpoint it loads; a catalog aggregates them into a manifest the product shows next to its software licenses.
A non-commercial entry must carry a restriction note."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass


@dataclass(frozen=True)
class WeightLicense:
    spdx_id: str
    name: str
    source_url: str
    attribution: str | None
    commercial_use: bool
    restriction: str | None = None

    def is_permissive(self) -> bool:
        return self.commercial_use

    def is_well_formed(self) -> bool:
        if not self.spdx_id.strip() or not self.name.strip() or not self.source_url.strip():
            return False
        if not self.commercial_use and not (self.restriction and self.restriction.strip()):
            return False
        return True


@dataclass(frozen=True)
class WeightLicenseEntry:
    provider_id: str
    license: WeightLicense


def weight_licenses_manifest_json(entries: list[WeightLicenseEntry]) -> str:
    bad = [e.provider_id for e in entries if not e.license.is_well_formed()]
    if bad:
        raise ValueError(f"malformed weight licenses for providers {bad}")
    rows = sorted(({"provider_id": e.provider_id, **asdict(e.license)} for e in entries), key=lambda r: r["provider_id"])
    return json.dumps({"model_weight_licenses": rows}, indent=2, sort_keys=True)


FLUX1_DEV = WeightLicense("LicenseRef-FLUX-1-dev-Non-Commercial", "FLUX.1 [dev] Non-Commercial License",
                          "https://huggingface.co/black-forest-labs/FLUX.1-dev", "Black Forest Labs", False,
                          "non-commercial use only; outputs may be used under the license's terms")
FLUX1_SCHNELL = WeightLicense("Apache-2.0", "Apache License 2.0", "https://huggingface.co/black-forest-labs/FLUX.1-schnell",
                              "Black Forest Labs", True)
LLAMA3 = WeightLicense("LicenseRef-Llama-3-Community", "Meta Llama 3 Community License",
                       "https://huggingface.co/meta-llama/Meta-Llama-3-8B", "Built with Meta Llama 3", True,
                       "acceptable-use policy applies; additional terms above 700M monthly active users")
