"""Tuning files, in the reference's formats (reference: tune/profile_config.py:59-74,
tune/search.py:70-102, tune/bandwidth.py:154-155, tool/generate_instances.py:20-25).

* ``configs/AlgoDict.pt``             ``{(TileM, TileN, TileK): Algo index}``
* ``configs/m{M}n{N}k{K}_{gpu}.json``  stage 1: lists ``BM, BN, dur, Algo`` (fastest GEMM
  tile configurations, ``dur`` in ms); stage 2: scalars ``BM, BN, dur, Algo`` plus
  ``hint`` (tile ids in slot order), ``cSeg`` (tiles per wave group) and ``rLDN``.
  This library adds optional keys (``raster_group``, ``two_stream_dur``, ``candidates_timed``,
  ``fused_dur``, ``stage1``) that the reference's readers ignore.  Stage 2 keeps the
  stage-1 lists under ``stage1`` so that a search can be re-run without re-profiling.
* ``configs/bandwidth_{op}_tp{ws}.pt`` / ``..._ws{ws}.pt``: float tensor ``[n, 2]`` of
  ``[elements, bus bandwidth in GB/s]``.
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Optional, Sequence

import torch

# Tile table of the native library, index = Algo (written by tool/generate_instances.py).
from ._algo_table import ALGO_TILES  # noqa: E402

REPO_ROOT = Path(__file__).resolve().parents[2]


def config_dir(path: Optional[os.PathLike] = None) -> Path:
    d = Path(path) if path is not None else Path(os.environ.get("FLASHOVERLAP_CONFIG_DIR", REPO_ROOT / "configs"))
    d.mkdir(parents=True, exist_ok=True)
    return d


def gpu_tag(name: Optional[str] = None) -> str:
    """Four-character GPU tag of the file names: characters 7..10 of the device
    name, lower case ("NVIDIA B200" -> "b200"), as the reference cuts it."""
    if name is None:
        name = torch.cuda.get_device_name() if torch.cuda.is_available() else "NVIDIA CPU0"
    return name[7:11].lower().strip() or "gpu"


def algo_dict() -> dict:
    return {tile: i for i, tile in enumerate(ALGO_TILES)}


def save_algo_dict(path: Optional[os.PathLike] = None) -> Path:
    f = config_dir(path) / "AlgoDict.pt"
    torch.save(algo_dict(), f)
    return f


def load_algo_dict(path: Optional[os.PathLike] = None) -> dict:
    f = config_dir(path) / "AlgoDict.pt"
    if not f.exists():
        return algo_dict()
    return torch.load(f, weights_only=False)


def json_path(M: int, N: int, K: int, path: Optional[os.PathLike] = None, gpu: Optional[str] = None) -> Path:
    return config_dir(path) / f"m{M}n{N}k{K}_{gpu or gpu_tag()}.json"


def save_stage1(M: int, N: int, K: int, BM: Sequence[int], BN: Sequence[int], dur: Sequence[float],
                Algo: Sequence[int], path=None, gpu=None, dur_raster: Optional[dict] = None) -> Path:
    """``dur_raster`` (optional, this library only): ``{raster group: [GEMM ms per
    listed configuration]}``, what the predictive search uses as the GEMM time
    of a (configuration, raster group) candidate."""
    if not (len(BM) == len(BN) == len(dur) == len(Algo)) or len(BM) == 0:
        raise ValueError("stage-1 lists must be non-empty and of equal length")
    f = json_path(M, N, K, path, gpu)
    data = {"BM": list(map(int, BM)), "BN": list(map(int, BN)), "dur": list(map(float, dur)),
            "Algo": list(map(int, Algo))}
    if dur_raster:
        for rg, col in dur_raster.items():
            if len(col) != len(BM):
                raise ValueError("dur_raster columns must be as long as the stage-1 lists")
        data["dur_raster"] = {str(int(rg)): [float(v) for v in col] for rg, col in dur_raster.items()}
    with open(f, "w", encoding="utf-8") as fh:
        json.dump(data, fh, indent=4)
    return f


def load_config(M: int, N: int, K: int, path=None, gpu=None) -> dict:
    f = json_path(M, N, K, path, gpu)
    if not f.exists():
        raise FileNotFoundError(f"{f} not found: profile the GEMM first (tune/profile_config.py)")
    try:
        with open(f, "r", encoding="utf-8") as fh:
            data = json.load(fh)
    except json.JSONDecodeError as exc:
        raise ValueError(f"{f} is not valid JSON: {exc}") from exc
    for key in ("BM", "BN", "dur", "Algo"):
        if key not in data:
            raise ValueError(f"{f} lacks the key {key!r}")
    return data


def stage1_lists(data: dict):
    """The stage-1 candidate lists of a config, whichever stage the file is in."""
    src = data
    if not isinstance(data["BM"], list):
        src = data.get("stage1")
        if src is None:  # a stage-2 file written by the reference: one candidate survives
            return [data["BM"]], [data["BN"]], [data["dur"]], [data["Algo"]]
    return list(src["BM"]), list(src["BN"]), list(src["dur"]), list(src["Algo"])


def stage1_raster_table(data: dict) -> dict:
    """``{raster group: [GEMM ms per stage-1 configuration]}`` if the profile recorded it, else {}."""
    src = data if isinstance(data["BM"], list) else (data.get("stage1") or {})
    return {int(rg): list(col) for rg, col in (src.get("dur_raster") or {}).items()}


def is_stage2(data: dict) -> bool:
    return all(k in data for k in ("hint", "cSeg")) and not isinstance(data["BM"], list)


def validate_stage2(data: dict, M: int, N: int) -> None:
    """Raise ValueError unless ``data`` is a consistent stage-2 solution for an M x N output."""
    if not is_stage2(data):
        raise ValueError("not a stage-2 config: run the search first (tune/search.py)")
    BM, BN = int(data["BM"]), int(data["BN"])
    if BM <= 0 or BN <= 0 or M % BM or N % BN:
        raise ValueError(f"tile {BM}x{BN} does not divide {M}x{N}")
    tiles = (M // BM) * (N // BN)
    hint, cseg = data["hint"], data["cSeg"]
    if len(hint) > tiles or sorted(set(hint)) != sorted(hint) or any(h < 0 or h >= tiles for h in hint):
        raise ValueError("hint must list distinct tile ids in [0, tiles)")
    if any(int(c) <= 0 for c in cseg) or sum(int(c) for c in cseg) != tiles:
        raise ValueError(f"cSeg must be positive and sum to the {tiles} tiles, got sum {sum(cseg)}")
    if int(data["Algo"]) < 0 or int(data["Algo"]) >= len(ALGO_TILES):
        raise ValueError("Algo index out of range")
    if tuple(ALGO_TILES[int(data["Algo"])][:2]) != (BM, BN):
        raise ValueError(f"Algo {data['Algo']} computes {ALGO_TILES[int(data['Algo'])][:2]} tiles, config says {BM}x{BN}")


def save_stage2(M: int, N: int, K: int, BM: int, BN: int, dur: float, Algo: int, hint: Sequence[int],
                cSeg: Sequence[int], path=None, gpu=None, **extra) -> Path:
    f = json_path(M, N, K, path, gpu)
    data = {}
    if f.exists():
        with open(f, "r", encoding="utf-8") as fh:
            data = json.load(fh)
    if isinstance(data.get("BM"), list):
        data["stage1"] = {k: data[k] for k in ("BM", "BN", "dur", "Algo", "dur_raster") if k in data}
        data.pop("dur_raster", None)
    data.update({"hint": [int(h) for h in hint], "cSeg": [int(c) for c in cSeg], "rLDN": 1, "BM": int(BM),
                 "BN": int(BN), "dur": float(dur), "Algo": int(Algo)})
    data.update(extra)
    validate_stage2(data, M, N)
    with open(f, "w", encoding="utf-8") as fh:
        json.dump(data, fh, indent=4)
    return f


def bandwidth_path(comm_op: str, world_size: int, multinode: bool = False, path=None) -> Path:
    return config_dir(path) / f"bandwidth_{comm_op}_{'ws' if multinode else 'tp'}{world_size}.pt"


def save_bandwidth(curve: torch.Tensor, comm_op: str, world_size: int, multinode: bool = False, path=None) -> Path:
    curve = torch.as_tensor(curve, dtype=torch.float32)
    if curve.dim() != 2 or curve.shape[1] != 2:
        raise ValueError("bandwidth curve must be [n, 2] = [elements, GB/s]")
    f = bandwidth_path(comm_op, world_size, multinode, path)
    torch.save(curve, f)
    return f


def load_bandwidth(comm_op: str, world_size: int, multinode: bool = False, path=None) -> torch.Tensor:
    f = bandwidth_path(comm_op, world_size, multinode, path)
    if not f.exists():
        raise FileNotFoundError(f"{f} not found: measure the curve first (tune/bandwidth.py)")
    return torch.load(f, weights_only=False)
