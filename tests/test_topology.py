"""Topology discovery from links, without devices: pair-link counting, level-0 shape, the matchers, and NVML queries against a
stand-in library that describes a box with one missing NVLink pair. (Reference behaviour: src/ops/op_common/topo/topo_host.cc:280-332
pair-link counter, :549-600 level-0 shape; matchers src/ops/op_common/topo/topo_match_*.h.)"""
import ctypes
import subprocess

import pytest

from hccl_b200._lib import lib

NONE, NVLINK, PCIE, SHM, NET = 0, 1, 2, 3, 4


def _topo(n, per_server, link, my_rank=0, match=0, active=None, nvls=1):
    m = (ctypes.c_uint8 * (n * n))(*[link(a, b) for a in range(n) for b in range(n)])
    act = (ctypes.c_uint32 * n)(*(active or [18] * n))
    desc, groups = ctypes.create_string_buffer(2048), ctypes.create_string_buffer(2048)
    fn = lib().HcclTopoFromLinks
    fn.argtypes = [ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_int, ctypes.c_char_p,
                   ctypes.c_uint32, ctypes.c_char_p, ctypes.c_uint32]
    rc = fn(n, per_server, m, act, nvls, my_rank, match, desc, len(desc), groups, len(groups))
    return rc, desc.value.decode(), [[int(x) for x in g.split(",")] for g in groups.value.decode().split("|") if g]


def test_full_nvswitch_box_counts_56_nvlink_pairs():
    rc, desc, groups = _topo(8, 8, lambda a, b: SHM if a == b else NVLINK)
    assert rc == 0
    assert "level0=NVSWITCH" in desc and "pairLinks[nvlink=56 pcie=0" in desc and "missing" not in desc
    assert "bw0=770" in desc                                  # 18 links x 50 GB/s x the measured copy efficiency
    assert groups == [list(range(8))]


def test_fewer_active_links_lower_the_bandwidth_weight():
    rc, desc, _ = _topo(8, 8, lambda a, b: SHM if a == b else NVLINK, active=[18] * 7 + [9])
    assert rc == 0 and "bw0=385" in desc                       # the slowest device bounds the level


def test_one_missing_link_is_named_and_demotes_the_shape():
    def link(a, b):
        if a == b:
            return SHM
        return NONE if {a, b} == {2, 5} else NVLINK
    rc, desc, _ = _topo(8, 8, link)
    assert rc == 0
    assert "level0=CLOS" in desc and "nvls=0" in desc and "missing=2-5" in desc and "none=2" in desc and "nvlink=54" in desc


def test_pcie_pair_makes_a_mesh_without_multicast():
    rc, desc, _ = _topo(4, 4, lambda a, b: SHM if a == b else (PCIE if {a, b} == {0, 3} else NVLINK))
    assert rc == 0 and "level0=MESH_1D" in desc and "nvls=0" in desc and "pcie=2" in desc and "bw0=55" in desc


def test_without_multicast_a_full_nvlink_box_is_a_mesh():
    rc, desc, _ = _topo(4, 4, lambda a, b: SHM if a == b else NVLINK, nvls=0)
    assert rc == 0 and "level0=MESH_1D" in desc


@pytest.mark.parametrize("rank", [0, 5, 11])
def test_multi_level_and_three_level_matchers(rank):
    link = lambda a, b: SHM if a == b else (NVLINK if a // 4 == b // 4 else NET)   # noqa: E731 - 3 servers x 4 GPUs
    rc, desc, g = _topo(12, 4, link, my_rank=rank, match=1)
    assert rc == 0 and "servers=3" in desc
    server = rank // 4
    assert g == [[server * 4 + i for i in range(4)], [rank % 4 + 4 * s for s in range(3)]]
    rc, _, g3 = _topo(12, 4, link, my_rank=rank, match=2)
    assert rc == 0 and g3[:2] == g and g3[2] == [rank]          # padded to exactly three levels


@pytest.mark.parametrize("n,rank,rows,cols", [(8, 5, 2, 4), (16, 6, 4, 4), (6, 4, 2, 3), (7, 3, 1, 7)])
def test_squeeze_2d_matcher_folds_a_flat_group(n, rank, rows, cols):
    rc, _, g = _topo(n, n, lambda a, b: SHM if a == b else NVLINK, my_rank=rank, match=3)
    assert rc == 0
    r, c = divmod(rank, cols)
    assert g == [[r * cols + j for j in range(cols)], [i * cols + c for i in range(rows)]]


def test_link_island_matcher_bridges_two_nvlink_islands():
    # GPUs 0-3 and 4-7 are NVLink islands, PCIe between them
    link = lambda a, b: SHM if a == b else (NVLINK if a // 4 == b // 4 else PCIE)   # noqa: E731
    rc, desc, g = _topo(8, 8, link, my_rank=6, match=4)
    assert rc == 0 and "level0=MESH_1D" in desc
    assert g == [[4, 5, 6, 7], [2, 6]]


FAKE_NVML = r"""
#include <string.h>
/* eight devices "0000:0N:00.0"; device 2 and device 5 have no NVLink path to each other; device 7 has 9 links up */
static int idx(const char *bus) { return bus[6] - '0'; }
int nvmlInit_v2(void) { return 0; }
int nvmlDeviceGetHandleByPciBusId_v2(const char *bus, void **dev) { if (strlen(bus) < 7 || idx(bus) < 0 || idx(bus) > 7) return 6; *dev = (void *)(long)(idx(bus) + 1); return 0; }
int nvmlDeviceGetP2PStatus(void *a, void *b, int cap, int *status) { long x = (long)a - 1, y = (long)b - 1; if (cap != 2) return 3; *status = ((x == 2 && y == 5) || (x == 5 && y == 2)) ? 2 : 0; return 0; }
int nvmlDeviceGetNvLinkState(void *a, unsigned link, int *active) { if (link >= 18) return 2; *active = ((long)a - 1 == 7) ? (link < 9) : 1; return 0; }
int nvmlDeviceGetNvLinkVersion(void *a, unsigned link, unsigned *v) { (void)a; (void)link; *v = 7; return 0; }
"""


def test_nvml_queries_against_a_stand_in_library(tmp_path, monkeypatch):
    src, so = tmp_path / "fake_nvml.c", tmp_path / "libfake_nvml.so"
    src.write_text(FAKE_NVML)
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", str(so), str(src)], check=True)
    monkeypatch.setenv("HCCL_NVML_LIB", str(so))
    probe = lib().HcclTopoProbeNvml
    probe.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_uint32)]

    def q(a, b):
        p2p, act, ver = ctypes.c_int(), ctypes.c_uint32(), ctypes.c_uint32()
        rc = probe(f"0000:0{a}:00.0".encode(), f"0000:0{b}:00.0".encode(), ctypes.byref(p2p), ctypes.byref(act), ctypes.byref(ver))
        return rc, p2p.value, act.value, ver.value

    assert q(0, 1) == (0, 1, 18, 7)
    assert q(2, 5) == (0, 0, 18, 7)              # the missing pair
    assert q(7, 0) == (0, 1, 9, 7)               # half of device 7's links are down
    # the matrix those answers give is the one-missing-link box of the test above
    def link(a, b):
        return SHM if a == b else (NVLINK if q(a, b)[1] == 1 else NONE)
    rc, desc, _ = _topo(8, 8, link, active=[q(a, (a + 1) % 8)[2] for a in range(8)])
    assert rc == 0 and "missing=2-5" in desc and "level0=CLOS" in desc
    monkeypatch.setenv("HCCL_NVML_LIB", str(tmp_path / "does_not_exist.so"))
    assert q(0, 1)[0] == 7                       # HCCL_E_UNAVAIL: no library, callers fall back to the runtime's attributes
