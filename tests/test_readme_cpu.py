"""The README's provider table names exactly the generator and trainer ids that the sm_100a bundle registers."""
import re
from pathlib import Path


def test_readme_lists_the_registered_generators_and_trainers():
    from inference_b200.media import provider_registry

    text = (Path(__file__).parent.parent / "README.md").read_text()
    rows = {line.split("|")[1].strip(): line.split("|")[2] for line in text.splitlines()
            if line.startswith("| ") and line.count("|") >= 3}
    listed = set(re.findall(r"`([a-z0-9_]+)`", rows["image generators"] + rows["video generator"]))
    reg = provider_registry("b200")
    assert listed == set(reg.ids("generator")), (listed ^ set(reg.ids("generator")))
    trainers = set(re.findall(r"`([a-z0-9_]+)`", rows["trainers"]))
    assert trainers == set(reg.ids("trainer")), (trainers ^ set(reg.ids("trainer")))
