"""Multi-rank path on CPU: two gloo ranks shard the token dimension, each quantizes its band with the
oracle (standing in for the kernel, which needs a GPU), and the concatenation of the ranks' outputs
equals the unsharded result byte for byte.  Also the partition arithmetic itself."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

from tilekernels_b200.sharding import shard_rows


@pytest.mark.parametrize('num_tokens,world,alignment', [(262144, 8, 128), (4096, 8, 128), (4001, 4, 128), (1000, 3, 128),
                                                        (100, 8, 128), (7168, 8, 128), (0, 2, 128), (4097, 2, 1)])
def test_shard_rows_partition(num_tokens, world, alignment):
    spans = [shard_rows(num_tokens, r, world, alignment) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == num_tokens
    for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
        assert a1 == b0 and a0 <= a1
    for start, stop in spans[:-1]:
        assert start % alignment == 0 and stop % alignment == 0
    sizes = [(b - a) // alignment for a, b in spans]
    assert max(sizes) - min(sizes) <= 1 + (num_tokens % alignment > 0)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, rows: int, result_dir: str) -> None:
    sys.path.insert(0, ROOT)
    import oracle
    from tilekernels_b200.sharding import shard_rows as shard
    from tilekernels_b200.testing import make_config_input
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    start, stop = shard(rows, rank, world, 4096)
    x = make_config_input('cfg5', stop - start, first_row=start)  # each rank generates only its own rows
    out, sf = oracle.cast(x, 'e4m3', (1, 128), round_sf=True, use_tma_aligned_col_major_sf=True, use_packed_ue8m0=True)
    # the data path has no collective; the only exchange is the timing reduction the benchmark does
    t = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.item() == world
    torch.save({'start': start, 'stop': stop, 'out': out.view(torch.uint8), 'sf': sf.contiguous()}, os.path.join(result_dir, f'rank{rank}.pt'))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsharded_cast(tmp_path, oracle):
    from tilekernels_b200.testing import make_config_input
    rows, world = 8192, 2
    mp.spawn(_rank_main, args=(world, _free_port(), rows, str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(os.path.join(tmp_path, f'rank{r}.pt')) for r in range(world)]
    x = make_config_input('cfg5', rows)
    out, sf = oracle.cast(x, 'e4m3', (1, 128), round_sf=True, use_tma_aligned_col_major_sf=True, use_packed_ue8m0=True)
    assert parts[0]['start'] == 0 and parts[0]['stop'] == parts[1]['start'] and parts[1]['stop'] == rows
    assert torch.equal(torch.cat([p['out'] for p in parts]), out.view(torch.uint8))
    assert torch.equal(torch.cat([p['sf'] for p in parts]), sf.contiguous())


def test_benchmark_shard_parity_check(oracle):
    """The check the benchmark runs on every rank (first and last 4096-row band of the shard against the CPU checker)
    accepts the correct outputs and rejects a single wrong code or scale byte in either band."""
    sys.path.insert(0, ROOT)
    import bench
    from tilekernels_b200.testing import make_config_input
    rows = 8192 + 512
    x = make_config_input('cfg5', rows)
    out, sf = oracle.cast(x, 'e4m3', (1, 128), round_sf=True, use_tma_aligned_col_major_sf=True, use_packed_ue8m0=True)
    assert bench.shard_parity(torch, oracle, x, out, sf, rows)
    bad = out.clone()
    bad.view(torch.uint8)[rows - 1, 7] ^= 1
    assert not bench.shard_parity(torch, oracle, x, bad, sf, rows)
    bad_sf = sf.clone()
    bad_sf[0, 0] += 1
    assert not bench.shard_parity(torch, oracle, x, out, bad_sf, rows)
