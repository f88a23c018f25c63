"""Child process of test_hostile_peer.py: honest clients connect to a fake server that replays mutated copies
of a real server's byte stream (recorded through a proxy). A client may get an error, a timeout or an odd
value; it must not crash or hang. Usage: mp_hostile_server.py <seed> <clients>."""
import asyncio
import os
import random
import socket
import struct
import sys
import threading
import time
from pathlib import Path

os.environ["EUX_SHM"] = "0"          # keep the frames on TCP, where the proxy can see them
sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import numpy as np  # noqa: E402

from execution_ucx_b200 import axon  # noqa: E402

to_client = bytearray()


def proxy(listener, target):
    inbound, _ = listener.accept()
    outbound = socket.create_connection(target)

    def pump(src, dst, record):
        try:
            while True:
                data = src.recv(65536)
                if not data:
                    break
                if record is not None:
                    record.extend(data)
                dst.sendall(data)
        except OSError:
            pass
        finally:
            try:
                dst.shutdown(socket.SHUT_WR)
            except OSError:
                pass

    threading.Thread(target=pump, args=(inbound, outbound, None), daemon=True).start()
    threading.Thread(target=pump, args=(outbound, inbound, to_client), daemon=True).start()


async def main(seed: int, clients: int) -> None:
    server = axon.AxonRuntime("real_srv", timeout=3000)

    async def scale(x: np.ndarray, k: int) -> np.ndarray:
        return x * k

    server.register_function(scale, from_dlpack_fn=np.from_dlpack)
    server.start_server()
    address = bytearray(server.get_local_address())
    port = struct.unpack_from("<H", address, 8)[0]
    listener = socket.socket()
    listener.bind(("127.0.0.1", 0))
    listener.listen(1)
    threading.Thread(target=proxy, args=(listener, ("127.0.0.1", port)), daemon=True).start()
    through_proxy = bytearray(address)
    struct.pack_into("<H", through_proxy, 8, listener.getsockname()[1])
    client = axon.AxonRuntime("recording_cli", timeout=3000)
    client.start_client()
    await client.connect_endpoint_async(bytes(through_proxy), "real_srv")
    small, big = np.arange(64, dtype=np.float32), np.arange(1 << 14, dtype=np.float32)
    for x in (small, small, big):
        assert np.array_equal(await client.invoke(x, 2, worker_name="real_srv", session_id=1, function="scale", from_dlpack_fn=np.from_dlpack), x * 2)
    client.stop()
    server.stop()
    await asyncio.sleep(0.2)
    stream = bytes(to_client)
    assert len(stream) > 60000, len(stream)

    rng = random.Random(seed)
    fake = socket.socket()
    fake.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    fake.bind(("127.0.0.1", 0))
    fake.listen(16)

    def answer(conn, data):
        try:
            conn.settimeout(0.3)
            try:
                conn.recv(65536)                      # the client's hello
            except OSError:
                pass
            cut = rng.randrange(40, 400)              # the answer in two pieces, the client's request read in between
            conn.sendall(bytes(data[:cut]))
            time.sleep(0.01)
            try:
                conn.recv(1 << 20)
            except OSError:
                pass
            conn.sendall(bytes(data[cut:]))
            time.sleep(0.05)
        except OSError:
            pass
        finally:
            try:
                conn.close()
            except OSError:
                pass

    def serve():
        while True:
            try:
                conn, _ = fake.accept()
            except OSError:
                return
            if rng.random() < 0.1:
                data = bytearray(rng.randbytes(rng.randrange(1, 400)))
            else:
                data = bytearray(stream)
                for _ in range(rng.randint(0, 8)):
                    j = rng.randrange(min(len(data), 1500)) if rng.random() < 0.7 else rng.randrange(len(data))
                    data[j] = rng.randrange(256) if rng.random() < 0.6 else (data[j] ^ (1 << rng.randrange(8)))
                if rng.random() < 0.3:
                    data = data[: rng.randrange(1, len(data))]
            threading.Thread(target=answer, args=(conn, data), daemon=True).start()

    threading.Thread(target=serve, daemon=True).start()
    fake_address = bytearray(address)
    struct.pack_into("<H", fake_address, 8, fake.getsockname()[1])
    outcomes = {}
    for i in range(clients):
        victim = axon.AxonRuntime("victim_%d" % i, timeout=300)
        victim.start_client()
        try:
            await asyncio.wait_for(victim.connect_endpoint_async(bytes(fake_address), "real_srv"), 2)
            y = await asyncio.wait_for(victim.invoke(small, 2, worker_name="real_srv", session_id=1, function="scale", from_dlpack_fn=np.from_dlpack), 2)
            kind = "answered" if isinstance(y, np.ndarray) else "odd"
        except Exception as e:
            kind = type(e).__name__
        outcomes[kind] = outcomes.get(kind, 0) + 1
        victim.stop()
    fake.close()
    print("outcomes", outcomes)


if __name__ == "__main__":
    asyncio.run(main(int(sys.argv[1]), int(sys.argv[2])))
    print("OK")
