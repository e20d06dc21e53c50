"""Validators of the checked mode (``APB_DEBUG_CHECKS=1``): bad tables are named on the host, good ones pass."""
import numpy as np
import pytest
import torch

from arctic_platform_b200.utils import checked
from arctic_platform_b200.utils.checked import TableError


def test_switch(monkeypatch):
    monkeypatch.delenv("APB_DEBUG_CHECKS", raising=False)
    checked.force(None)
    assert not checked.enabled() and not checked.active_for(torch.zeros(1))
    monkeypatch.setenv("APB_DEBUG_CHECKS", "1")
    assert checked.enabled() and checked.active_for(torch.zeros(1))
    checked.force(False)
    assert not checked.enabled()
    checked.force(None)


def test_ranges_and_masks():
    checked.check_range("t", torch.tensor([[0, 3], [2, 1]]), 0, 4)
    with pytest.raises(TableError, match=r"t\[1, 0\] = 7 outside \[0, 4\)"):
        checked.check_range("t", torch.tensor([[0, 3], [7, 1]]), 0, 4)
    checked.check_range("t", torch.tensor([[0, 3], [7, 1]]), 0, 4, where=torch.tensor([True, False]))      # masked row
    checked.check_range("t", np.zeros((0,), dtype=np.int32), 0, 1)


def test_cu_seqlens():
    checked.check_cu_seqlens(torch.tensor([0, 3, 3, 9]), 9)
    for cu, needle in ((torch.tensor([1, 3]), "start at 0"), (torch.tensor([0, 5, 4]), "smaller"), (torch.tensor([0, 5]), "holds 6")):
        with pytest.raises(TableError, match=needle):
            checked.check_cu_seqlens(cu, 6)


def test_page_tables():
    tab = torch.tensor([[3, 4, 0, 0], [5, 99, 0, 0], [1, 2, 6, 7]], dtype=torch.int32)
    checked.check_page_table("pt", tab, torch.tensor([20, 16, 64]), num_pages=8)          # 99 sits beyond row 1's pages
    with pytest.raises(TableError, match=r"pt\[1, 1\] = 99"):
        checked.check_page_table("pt", tab, torch.tensor([20, 17, 64]), num_pages=8)
    with pytest.raises(TableError, match="5 pages"):
        checked.check_page_table("pt", tab, torch.tensor([20, 16, 65]), num_pages=8)
    checked.check_page_table("pt", tab, torch.tensor([20, 17, 65]), num_pages=8, active=torch.tensor([1, 0, 0]))
    with pytest.raises(TableError, match="negative"):
        checked.check_page_table("pt", tab, torch.tensor([20, -1, 64]), num_pages=8)


def test_forest_tables_from_the_planner_pass_and_corruptions_are_named():
    from arctic_platform_b200.ops.forest_attention import ForestNode, plan_forest
    nodes = [ForestNode(0, range(0, 8), np.arange(0, 4, dtype=np.int32), 60),
             ForestNode(1, range(0, 4), np.arange(4, 6, dtype=np.int32), 32),
             ForestNode(1, range(4, 8), np.arange(6, 8, dtype=np.int32), 20)]
    qs, qc, pg, ln, lv, _mask, G, nl, _s, _c = plan_forest(nodes, num_slots=8, max_pages=6, max_rows=128)
    checked.check_forest(qs, qc, pg, ln, lv, num_slots=8, num_pages=8, n_levels=nl)
    with pytest.raises(TableError, match="exceed the batch"):
        checked.check_forest(qs, qc, pg, ln, lv, num_slots=6, num_pages=8, n_levels=nl)
    with pytest.raises(TableError, match=r"forest.pages\[2, 1\] = 7"):
        checked.check_forest(qs, qc, pg, ln, lv, num_slots=8, num_pages=7, n_levels=nl)
    bad = lv.copy()
    bad[1] = 2
    with pytest.raises(TableError, match="forest.level"):
        checked.check_forest(qs, qc, pg, ln, bad, num_slots=8, num_pages=8, n_levels=nl)
    long = ln.copy()
    long[0] = 16 * 6 + 1
    with pytest.raises(TableError, match="7 pages"):
        checked.check_forest(qs, qc, pg, long, lv, num_slots=8, num_pages=8, n_levels=nl)


def test_routing_tile_maps_and_copy_tables():
    checked.check_routing(torch.tensor([0, -1, 3]), torch.tensor([5, 10**6, 0]), world=4, rows_cap=8)
    with pytest.raises(TableError, match="dst_rank"):
        checked.check_routing(torch.tensor([0, 4]), torch.tensor([0, 0]), world=4, rows_cap=8)
    with pytest.raises(TableError, match=r"dst_row\[0\] = 8"):
        checked.check_routing(torch.tensor([1]), torch.tensor([8]), world=4, rows_cap=8)
    tm = torch.tensor([[0, 0, 0, 0], [1, 2, 0, 0], [9, 9, 0, 0]])
    checked.check_tile_map(tm, 2, groups=2, m_tiles_cap=3)
    with pytest.raises(TableError, match="group"):
        checked.check_tile_map(tm, 3, groups=2, m_tiles_cap=3)
    with pytest.raises(TableError, match="announced"):
        checked.check_tile_map(tm, 4, groups=2, m_tiles_cap=3)
    checked.check_copy_table("sync", [0, 10], [5, 0], [5, 5], src_size=15, dst_size=10)
    with pytest.raises(TableError, match="source"):
        checked.check_copy_table("sync", [0, 11], [5, 0], [5, 5], src_size=15, dst_size=10)
    with pytest.raises(TableError, match="overlap"):
        checked.check_copy_table("sync", [0, 10], [4, 0], [5, 5], src_size=15, dst_size=10)
    with pytest.raises(TableError, match="destination"):
        checked.check_copy_table("sync", [0], [8], [5], src_size=15, dst_size=10)


def test_hooks_fire_only_in_checked_mode():
    from arctic_platform_b200.ops.attention import AttnLayout
    from arctic_platform_b200.ops.forest_attention import ForestNode, build_forest_tables
    checked.force(False)
    try:
        AttnLayout.from_cu_seqlens([0, 5, 3])                 # unchecked: the table is taken as given
        checked.force(True)
        with pytest.raises(TableError, match="smaller"):
            AttnLayout.from_cu_seqlens([0, 5, 3])
        assert AttnLayout.from_cu_seqlens([0, 5, 9]).total_tokens == 9
        good = [ForestNode(0, range(0, 4), np.arange(2, dtype=np.int32), 30)]
        assert build_forest_tables(good, 4, 4, 128, "cpu").n_nodes == 1
        with pytest.raises(TableError, match="exceed the batch"):
            build_forest_tables([ForestNode(0, range(2, 6), np.arange(2, dtype=np.int32), 30)], 4, 4, 128, "cpu")
    finally:
        checked.force(None)
