"""Pass one file descriptor per rank to every other rank of the node.

CUDA virtual-memory allocations are shared between processes as POSIX file descriptors, and
a descriptor only crosses a process boundary as ``SCM_RIGHTS`` ancillary data of a Unix
socket.  Every rank listens on an abstract-namespace socket whose name is spread with the
control plane, serves its descriptor to whoever connects, and fetches the others'.
"""

from __future__ import annotations

import os
import socket
import threading
import uuid


def exchange_fds(control, my_fd: int, timeout_s: float = 120.0) -> list[int]:
    """Returns ``fds[peer]`` for every rank (``fds[rank]`` is ``my_fd`` itself)."""
    rank, size = control.rank, control.size
    directory = os.environ.get("AFDEP_SOCKET_DIR")
    token = uuid.uuid4().hex
    if directory:
        name = os.path.join(directory, f"afdep-{token}-{rank}.sock")
    else:
        name = f"\0afdep-{token}-{rank}"
    server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    server.bind(name)
    server.listen(size)
    server.settimeout(timeout_s)
    names = control.all_gather(name)   # every server is listening once this returns
    errors: list[BaseException] = []

    def serve() -> None:
        try:
            for _ in range(size - 1):
                conn, _ = server.accept()
                with conn:
                    conn.settimeout(timeout_s)
                    conn.recv(1)
                    socket.send_fds(conn, [b"f"], [my_fd])
        except BaseException as exc:  # noqa: BLE001 - re-raised on the caller's thread
            errors.append(exc)

    thread = threading.Thread(target=serve, daemon=True)
    thread.start()
    fds = [-1] * size
    fds[rank] = my_fd
    try:
        for peer in range(size):
            if peer == rank:
                continue
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as client:
                client.settimeout(timeout_s)
                client.connect(names[peer])
                client.send(b"r")
                _, received, _, _ = socket.recv_fds(client, 16, 1)
                if len(received) != 1:
                    raise RuntimeError(f"rank {peer} did not send its heap descriptor")
                fds[peer] = received[0]
        thread.join(timeout_s)
        if errors:
            raise RuntimeError(f"descriptor exchange failed: {errors[0]}")
    finally:
        server.close()
        if directory:
            try:
                os.unlink(name)
            except OSError:
                pass
    control.barrier()
    return fds
