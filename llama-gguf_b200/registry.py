"""Model registry: what a path holds -> the loader that makes a context of it.

  * a .gguf file: `general.architecture` picks the transformer family inside the library (GpuOnlyInference.from_gguf);
  * a folder with config.json: its "architecture" picks a module of this package that turns the config into a layer program and
    feeds model.safetensors (LOADERS below)."""
import json
import os

from . import GpuOnlyInference, Unsupported


def _lazilorn(path, **kw):
    from . import lazilorn
    return lazilorn.load(path, **kw)


def _mefurax(path, **kw):
    from . import mefurax
    return mefurax.load(path, **kw)


def _madudra(path, **kw):
    from . import madudra
    return madudra.load(path, **kw)


def _marosun(path, **kw):
    from . import marosun
    return marosun.load(path, **kw)


LOADERS = {"Lazilorn": _lazilorn, "Mefurax": _mefurax, "Madudra": _madudra, "Marosun": _marosun}


def architecture_of(path):
    if os.path.isdir(path):
        with open(os.path.join(path, "config.json")) as f:
            return json.load(f).get("architecture")
    from . import GgufFile
    with GgufFile(path) as f:
        return f.architecture()


def load_model(path, max_seq_len=4096, max_batch=8, compute="bfloat16", device=0, **kw):
    """A context for the model at `path`, chosen by what the path holds."""
    if os.path.isdir(path):
        arch = architecture_of(path)
        if arch not in LOADERS:
            raise Unsupported(f"{path}: architecture {arch!r} is not registered (known: {sorted(LOADERS)})")
        return LOADERS[arch](path, max_seq_len=max_seq_len, max_batch=max_batch, compute=compute, device=device, **kw)
    if compute != "bfloat16" and compute is not None:
        raise Unsupported("GGUF models run in their quantised types; `compute` applies to safetensors models")
    return GpuOnlyInference.from_gguf(path, max_seq_len=max_seq_len, max_batch=max_batch, device=device, **kw)
