"""Energy server: molecular geometries in, ANI energy and gradient out, over a TCP socket.

The wire format is the reference's (``energy_server.py:131-187``, ``client_server.py``,
``energy_client.py``): the client sends one UTF-8 JSON text ``{"X": [[type, x, y, z], ...]}``
(compacted element ids H 0, C 1, N 2, O 3; coordinates in Angstrom) of at most 1 MiB in one
message, and receives ``{"energy": E, "gradient": [g0, g1, ...]}`` -- E in Hartree including the
atomic self energies, the gradient flattened atom by atom (x, y, z) in Hartree/Bohr.  A
connection serves requests until the client closes it.

The reference evaluates each request with a float64 CPU trainer through ``predict`` and
``coordinate_gradients``; here the evaluator is any object with those two methods -- a
``TrainerMultiTower`` on one GPU by default -- so the protocol can be tested without a GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import socket

import numpy as np

from .data.dataset import RawDataset

ENCODING = "utf-8"
MAX_BYTES = 1024 ** 2        # one request or response is read with a single recv of this size
BACKLOG = 10
BOHR = 0.52917721092         # Angstrom per Bohr (energy_server.py: the gradient is sent in Hartree/Bohr)
# Atomic self energies (Hartree) that the training targets had subtracted, wB97X/6-31G(d)
# (data_utils.py:28-33 of the reference): doublet H, triplet C, quartet N, triplet O.
SELF_ENERGY = (-0.49932123901, -37.83271996200, -54.57325122225, -75.04147134502)


def evaluate(evaluator, X) -> dict:
    """Energy (Hartree, self energies included) and gradient (Hartree/Bohr, flattened) of one geometry."""
    arr = np.asarray(X, dtype=np.float64)
    if arr.ndim != 2 or arr.shape[1] != 4 or arr.shape[0] == 0:
        raise ValueError("X must be a non-empty list of [type, x, y, z]")
    types = arr[:, 0].astype(np.int64)
    if np.any(types != arr[:, 0]) or types.min() < 0 or types.max() > 3:
        raise ValueError("element ids must be 0 (H), 1 (C), 2 (N) or 3 (O)")
    rd = RawDataset([arr], [0.0])
    energy = float(evaluator.predict(rd)[0]) + float(sum(SELF_ENERGY[t] for t in types))
    gradient = np.asarray(list(evaluator.coordinate_gradients(rd))[0], dtype=np.float64).reshape(-1)
    return {"energy": energy, "gradient": [float(g) * BOHR for g in gradient]}


def handle_request(evaluator, text: str) -> str:
    """One request text -> one response text.  A malformed request gets ``{"error": ...}`` instead of
    killing the server (the reference would raise and die)."""
    try:
        return json.dumps(evaluate(evaluator, json.loads(text).get("X")))
    except Exception as exc:   # the client sees what was wrong; the server keeps serving
        return json.dumps({"error": f"{type(exc).__name__}: {exc}"})


def serve(evaluator, host: str = "127.0.0.1", port: int = 5000, max_connections: int | None = None,
          ready=None, debug: bool = False) -> None:
    """Blocking accept loop.  ``max_connections`` ends it after that many connections (tests);
    ``ready`` (a ``threading.Event``) is set once the socket listens."""
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        s.bind((host, port))
        s.listen(BACKLOG)
        if ready is not None:
            ready.set()
        served = 0
        while max_connections is None or served < max_connections:
            conn, addr = s.accept()
            served += 1
            with conn:
                if debug:
                    print(f"connection from {addr}")
                while True:
                    data = conn.recv(MAX_BYTES)
                    if not data:
                        break
                    conn.sendall(handle_request(evaluator, data.decode(ENCODING)).encode(ENCODING))


def request(host: str, port: int, X) -> dict:
    """What ``energy_client.py`` does: send one geometry, return the decoded answer."""
    with socket.create_connection((host, port)) as s:
        s.sendall(json.dumps({"X": [list(map(float, row)) for row in X]}).encode(ENCODING))
        return json.loads(s.recv(MAX_BYTES).decode(ENCODING))


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description="ANI energy + gradient server (khan's energy_server.py protocol)")
    ap.add_argument("--save-dir", required=True, help="directory holding save_file.npz (khan checkpoint)")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=5000)
    ap.add_argument("--activation-function", default="celu")
    ap.add_argument("--precision", default="float64", choices=["float32", "float64"],
                    help="the reference serves in float64; float32 takes the fused tensor-core networks")
    ap.add_argument("--debug", action="store_true")
    args = ap.parse_args(argv)

    import torch

    from .model import activations
    from .training.trainer_multi_tower import TrainerMultiTower
    save_file = os.path.join(args.save_dir, "save_file.npz")
    if not os.path.exists(save_file):
        raise IOError("Saved NN numpy file does not exist")
    trainer = TrainerMultiTower(None, [torch.device("cuda", torch.cuda.current_device())],
                                precision=args.precision, layer_sizes=(128, 128, 64, 1),
                                activation_fn=activations.get_fn_by_name(args.activation_function))
    trainer.load_numpy(save_file, strict=False)
    if args.debug:
        print(f"Server listening on port {args.port}")
    serve(trainer, args.host, args.port, debug=args.debug)


if __name__ == "__main__":
    main()
