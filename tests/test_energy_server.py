"""Protocol of the energy server (the reference's energy_server.py / energy_client.py exchange) with a
stand-in evaluator, on the CPU: JSON {X} in, {energy, gradient} out, Hartree and Hartree/Bohr, self
energies added, several requests per connection, malformed requests answered instead of fatal."""
import json
import socket
import threading

import numpy as np

from khan_b200 import energy_server as es


class _Harmonic:
    """E = sum |x|^2 over atoms; dE/dx = 2 x."""

    def predict(self, rd):
        return [float((m[:, 1:] ** 2).sum()) for m in rd.all_Xs]

    def coordinate_gradients(self, rd):
        for m in rd.all_Xs:
            yield 2.0 * m[:, 1:]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_evaluate_units_and_self_energies():
    X = [[1, 0.1, 0.2, 0.3], [0, -1.0, 0.5, 0.0], [3, 0.0, 0.0, 2.0]]
    out = es.evaluate(_Harmonic(), X)
    coords = np.array(X)[:, 1:]
    want_e = (coords ** 2).sum() + es.SELF_ENERGY[1] + es.SELF_ENERGY[0] + es.SELF_ENERGY[3]
    assert abs(out["energy"] - want_e) < 1e-12
    np.testing.assert_allclose(out["gradient"], (2.0 * coords).reshape(-1) * es.BOHR, rtol=1e-15)
    assert len(out["gradient"]) == 9 and all(isinstance(g, float) for g in out["gradient"])


def test_requests_over_a_socket_and_bad_input():
    port, ready = _free_port(), threading.Event()
    th = threading.Thread(target=es.serve, args=(_Harmonic(), "127.0.0.1", port),
                          kwargs={"max_connections": 2, "ready": ready}, daemon=True)
    th.start()
    assert ready.wait(10)
    X = [[0, 0.0, 0.0, 0.37], [0, 0.0, 0.0, -0.37]]
    ans = es.request("127.0.0.1", port, X)
    assert abs(ans["energy"] - (2 * 0.37 ** 2 + 2 * es.SELF_ENERGY[0])) < 1e-12
    # one connection, three messages: a good one, an element id out of range, not JSON at all
    with socket.create_connection(("127.0.0.1", port)) as s:
        for text, check in ((json.dumps({"X": X}), lambda a: len(a["gradient"]) == 6),
                            (json.dumps({"X": [[7, 0, 0, 0]]}), lambda a: "element ids" in a["error"]),
                            ("not json", lambda a: "error" in a)):
            s.sendall(text.encode())
            assert check(json.loads(s.recv(es.MAX_BYTES).decode()))
    th.join(10)
    assert not th.is_alive()
