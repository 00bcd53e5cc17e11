"""Out-of-core DARLIN: column blocks streamed from pinned host memory give the in-memory result."""
import pytest
import torch

from parameter_server_b200.data.synthetic import zipf_sparse_matrix

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("binary", [False, True])
def test_streamed_blocks_match_in_memory(binary):
    from parameter_server_b200.models.darlin import DarlinConfig, DarlinSolver
    from parameter_server_b200.parallel.peer import PeerGroup

    off, idx, vals, y, _ = zipf_sparse_matrix(3000, 4096, 20, seed=4, device="cuda", binary=binary, zipf_s=0.9)
    cfg = dict(lambda1=0.3, max_pass=4, feature_block_ratio=1.0, seed=1)
    runs = []
    for ooc in (False, True):
        sol = DarlinSolver(PeerGroup.single(torch.device("cuda", 0)), DarlinConfig(**cfg), out_of_core=ooc, prefetch_depth=3)
        sol.preprocess(off, idx * 31 + 5, vals, y)
        runs.append((sol.run(), sol))
    (p0, s0), (p1, s1) = runs
    per_pass = -(-s1.nblk // s1.blocks_per_launch)          # one launch per batch of streamed blocks
    assert s1.nblk > s1.blocks_per_launch and s1.h2d_bytes > 0
    assert s1.kernel_launches == 4 * per_pass and s0.kernel_launches == 4
    for a, b in zip(p0, p1):
        assert b.objv == pytest.approx(a.objv, rel=1e-4) and abs(a.nnz_w - b.nnz_w) <= 2
    s1.check_status()


def test_streamed_blocks_with_bounded_delay():
    """Batches of streamed blocks are whole synchronisation groups (max_block_delay + 1 blocks)."""
    from parameter_server_b200.models.darlin import DarlinConfig, DarlinSolver
    from parameter_server_b200.parallel.peer import PeerGroup

    off, idx, vals, y, _ = zipf_sparse_matrix(3000, 4096, 20, seed=4, device="cuda", zipf_s=0.9)
    cfg = dict(lambda1=0.3, max_pass=3, feature_block_ratio=1.0, seed=1, max_block_delay=2)
    runs = []
    for ooc in (False, True):
        sol = DarlinSolver(PeerGroup.single(torch.device("cuda", 0)), DarlinConfig(**cfg), out_of_core=ooc, prefetch_depth=2,
                           blocks_per_launch=4)
        sol.preprocess(off, idx * 31 + 5, vals, y)
        runs.append((sol.run(), sol))
    (p0, _), (p1, s1) = runs
    assert s1.blocks_per_launch == 6
    for a, b in zip(p0, p1):
        assert b.objv == pytest.approx(a.objv, rel=1e-4)
    s1.check_status()
