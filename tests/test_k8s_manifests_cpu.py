"""The Kubernetes manifests parse, ask for the node's eight GPUs, and name scripts and flags that exist."""
import glob
import os
import re

import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _containers(doc):
    return doc["spec"]["template"]["spec"]["containers"]


def test_manifests_reference_existing_scripts_and_flags():
    files = sorted(glob.glob(os.path.join(ROOT, "k8s", "*.yaml")))
    assert len(files) >= 3
    from jax_gpt_b200.trainer.config import TrainConfig
    train_fields = set(TrainConfig.__dataclass_fields__)
    for f in files:
        doc = yaml.safe_load(open(f))
        assert doc["kind"] == "Job" and doc["spec"]["backoffLimit"] == 0
        for c in _containers(doc):
            assert c["resources"]["limits"]["nvidia.com/gpu"] == 8
            assert any(m["mountPath"] == "/dev/shm" for m in c["volumeMounts"])
            text = " ".join(c.get("command", []) + [str(a) for a in c.get("args", [])])
            assert "--master-addr" in text and "127.0.0.1" in text      # single-pod rendezvous on loopback
            for script in re.findall(r"(scripts/\w+\.py|bench\.py)", text):
                assert os.path.exists(os.path.join(ROOT, script)), (f, script)
            if "scripts/train.py" in text:
                src = open(os.path.join(ROOT, "scripts", "train.py")).read()
                for flag in re.findall(r"--(\w+)=", text.split("scripts/train.py", 1)[1]):
                    assert flag in train_fields or f'"--{flag}"' in src, (f, flag)
            if "scripts/eval_humaneval.py" in text:
                src = open(os.path.join(ROOT, "scripts", "eval_humaneval.py")).read()
                for flag in re.findall(r"--([\w-]+)=", text.split("scripts/eval_humaneval.py", 1)[1]):
                    assert f'"--{flag}"' in src, (f, flag)
            if "scripts/bench_prefill_decode.py" in text:
                src = open(os.path.join(ROOT, "scripts", "bench_prefill_decode.py")).read()
                tail = text.split("scripts/bench_prefill_decode.py", 1)[1]
                for flag in re.findall(r"--([\w-]+)", tail):
                    assert f'"--{flag}"' in src, (f, flag)
