"""The library is called from two host threads at once (autograd runs the unpack hooks on its own thread while the
forward thread keeps packing) and on several streams: results must not depend on it."""
import threading

import pytest
import torch

import oracle
from helpers import assert_bits_equal

pytestmark = pytest.mark.gpu


def test_two_threads_two_streams_give_the_serial_results():
    from gact.ops import quantize_pack, dequantize_and_unpack
    cases = []
    for i, (dtype, bits, n) in enumerate([(torch.float16, 2, 256 * 3000 + 7), (torch.bfloat16, 4, 256 * 2048),
                                           (torch.float32, 8, 100 * 77), (torch.float16, 1, 256 * 4096 + 300),
                                           (torch.float32, 2, 256 * 1999), (torch.bfloat16, 8, 256 * 777 + 5)]):
        g = torch.Generator().manual_seed(i)
        cases.append((torch.randn(n, generator=g).to(dtype).cuda(), bits, 100 + i))
    serial = []
    for x, bits, seed in cases:
        q, sc, mn = quantize_pack(x, bits, seed, rng_mode="fast")
        serial.append((q.clone(), sc.clone(), mn.clone(), dequantize_and_unpack(q, (x.numel(),), bits, sc, mn).clone()))
    torch.cuda.synchronize()

    results = [None] * len(cases)
    errors = []

    def worker(idx_list):
        try:
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                for _ in range(20):                      # keep both threads launching at the same time for a while
                    for i in idx_list:
                        x, bits, seed = cases[i]
                        q, sc, mn = quantize_pack(x, bits, seed, rng_mode="fast")
                        y = dequantize_and_unpack(q, (x.numel(),), bits, sc, mn)
                        results[i] = (q, sc, mn, y)
            stream.synchronize()
        except Exception as e:                           # surfaced by the main thread
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(ids,)) for ids in ([0, 2, 4], [1, 3, 5])]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    torch.cuda.synchronize()
    for i, (want, got) in enumerate(zip(serial, results)):
        assert torch.equal(want[0][:-1], got[0][:-1]), i      # the spare last byte is unspecified
        for a, b, what in ((want[1], got[1], "scale"), (want[2], got[2], "min"), (want[3], got[3], "dequantized")):
            assert_bits_equal(b.reshape(-1), a.reshape(-1), f"{what} case {i}")
