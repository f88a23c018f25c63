"""Child process of test_hostile_peer.py: a server runtime is sent mutated copies of a legitimate client's
TCP byte stream (recorded through a proxy), and random bytes. It must neither crash nor hang, and a legitimate
client must still be served in between. Usage: mp_hostile_peer.py <seed> <attacks>."""
import asyncio
import os
import random
import socket
import struct
import sys
import threading
from pathlib import Path

os.environ["EUX_SHM"] = "0"          # keep the frames on TCP, where the proxy can see them
sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import numpy as np  # noqa: E402

from execution_ucx_b200 import axon  # noqa: E402

recorded = bytearray()


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

    threading.Thread(target=pump, args=(inbound, outbound, recorded), daemon=True).start()
    threading.Thread(target=pump, args=(outbound, inbound, None), daemon=True).start()


async def main(seed: int, attacks: int) -> None:
    server = axon.AxonRuntime("hostile_srv", timeout=3000)

    async def scale(x: np.ndarray, k: int) -> np.ndarray:
        return x * k

    server.register_function(scale, from_dlpack_fn=np.from_dlpack)
    server.start_server()
    address = bytes(server.get_local_address())
    _magic, _ipv4, port = struct.unpack_from("<IIH", address, 0)
    listener = socket.socket()
    listener.bind(("127.0.0.1", 0))
    listener.listen(1)
    threading.Thread(target=proxy, args=(listener, ("127.0.0.1", port)), daemon=True).start()
    through_proxy = bytearray(address)
    struct.pack_into("<H", through_proxy, 8, listener.getsockname()[1])
    client = axon.AxonRuntime("hostile_cli", timeout=3000)
    client.start_client()
    await client.connect_endpoint_async(bytes(through_proxy), "hostile_srv")
    small, big = np.arange(64, dtype=np.float32), np.arange(1 << 14, dtype=np.float32)   # eager and rendezvous
    for x in (small, small, big):
        y = await client.invoke(x, 2, worker_name="hostile_srv", session_id=1, function="scale", from_dlpack_fn=np.from_dlpack)
        assert np.array_equal(y, x * 2)
    client.stop()
    await asyncio.sleep(0.2)
    stream = bytes(recorded)
    assert len(stream) > 60000, len(stream)
    rng = random.Random(seed)
    loop = asyncio.get_running_loop()

    def attack():
        if rng.random() < 0.15:
            data = bytearray(rng.randbytes(rng.randrange(1, 400)))
        else:
            data = bytearray(stream)
            for _ in range(rng.randint(1, 8)):
                # most of the control information sits in the first frames
                j = rng.randrange(min(len(data), 1500)) if rng.random() < 0.7 else rng.randrange(len(data))
                data[j] = rng.randrange(256) if rng.random() < 0.6 else (data[j] ^ (1 << rng.randrange(8)))
            if rng.random() < 0.3:
                data = data[: rng.randrange(1, len(data))]
        with socket.create_connection(("127.0.0.1", port), timeout=5) as s:
            s.settimeout(0.05)
            s.sendall(bytes(data))
            try:
                s.recv(4096)
            except OSError:
                pass

    for i in range(attacks):
        await loop.run_in_executor(None, attack)
        if i % 100 == 99 or i == attacks - 1:
            honest = axon.AxonRuntime("hostile_cli_%d" % i, timeout=3000)
            honest.start_client()
            await honest.connect_endpoint_async(address, "hostile_srv")
            y = await honest.invoke(small, 3, worker_name="hostile_srv", session_id=2, function="scale", from_dlpack_fn=np.from_dlpack)
            assert np.array_equal(y, small * 3)
            honest.stop()
    print("refused", server.transport_stats()["frames_refused"])
    server.stop()


if __name__ == "__main__":
    asyncio.run(main(int(sys.argv[1]), int(sys.argv[2])))
    print("OK")
