"""The cut of the keys for decode attention (``parts.attention.cut_keys``) against a table of what a B200
holds in thread-block clusters of each size: no GPU needed."""
import pytest

from llm_rs_b200.parts.attention import CAPACITY_USED, FIXED_KEYS, LIGHT_COST, MAX_CLUSTER, cut_keys, cut_keys_and_ring

# Blocks of the decode kernel (heads of 128, 4 query heads per key head) that a B200 holds in clusters of 1..16.
B200 = [296, 296, 279, 284, 280, 270, 259, 264, 270, 260, 231, 252, 221, 196, 210, 224]


def held(cluster):
    return B200[cluster - 1]


def splits_of(length, keys):
    return -(-length // keys)


@pytest.mark.parametrize("requests,splits", [
    (1, 16), (2, 13), (3, 10), (4, 8), (5, 6), (6, 5), (7, 4), (8, 4), (9, 3), (10, 3), (11, 3), (16, 2), (17, 2), (18, 2),
    (32, 1), (64, 1)])
def test_splits_at_a_context_of_4096(requests, splits):
    """Eight key heads a request: one wave of blocks where one exists, as many splits as fit it."""
    keys = cut_keys(4096, requests * 8, held)
    assert keys % 64 == 0 and splits_of(4096, keys) == splits
    if requests <= 36:
        assert splits * requests * 8 <= CAPACITY_USED * held(splits)


def test_a_second_wave_is_taken_when_it_is_cheaper():
    # 12 requests: three splits would be 288 blocks in clusters of 3, of which the device holds 279; two
    # splits of 2,048 keys in one wave cost 2,240, five splits of 832 keys in two waves 2,048.
    assert splits_of(4096, cut_keys(4096, 12 * 8, held)) == 5
    # 20 requests: one split costs 4,288, three splits in two waves 3,200, five splits in three waves 3,072.
    assert splits_of(4096, cut_keys(4096, 20 * 8, held)) == 5


def test_a_full_wave_is_not_trusted():
    # 7 requests x 8 heads x 5 splits = 280 blocks is all the device holds in clusters of 5: measured as two waves.
    assert splits_of(4096, cut_keys(4096, 7 * 8, held)) == 4


def test_few_requests_with_long_contexts_take_the_merging_kernel():
    keys = cut_keys(32768, 8, held)               # one request: 37 splits of 896 keys
    assert splits_of(32768, keys) > MAX_CLUSTER and keys <= 2048 and keys % 64 == 0
    keys = cut_keys(32768, 8 * 8, held)           # eight requests stay with the cluster
    assert splits_of(32768, keys) <= MAX_CLUSTER


@pytest.mark.parametrize("length", [1, 63, 64, 100, 129, 1000, 4097, 40000])
@pytest.mark.parametrize("units", [1, 8, 40, 64, 300, 1000])
def test_every_cut_is_the_cheapest_of_its_kind(length, units):
    keys = cut_keys(length, units, held)
    assert keys % 64 == 0 and keys >= 128
    splits = splits_of(length, keys)
    if splits <= MAX_CLUSTER:
        costs = []
        for s in range(1, MAX_CLUSTER + 1):
            k = max(-(-(-(-length // s)) // 64) * 64, 128)
            real = splits_of(length, k)
            costs.append(-(-(real * units) // int(CAPACITY_USED * held(real))) * (k + FIXED_KEYS))
        assert -(-(splits * units) // int(CAPACITY_USED * held(splits))) * (keys + FIXED_KEYS) == min(costs)


# The same for the kernel with the ring of two tiles per warp, of which three blocks fit an SM.
B200_LIGHT = [444, 444, 420, 424, 420, 408, 392, 400, 396, 390, 352, 372, 338, 294, 315, 336]


def held_light(cluster):
    return B200_LIGHT[cluster - 1]


@pytest.mark.parametrize("requests,ring", [(8, 3), (32, 3), (36, 3), (38, 2), (40, 2), (48, 2), (54, 2), (56, 3), (64, 3)])
def test_the_light_kernel_is_taken_where_it_saves_a_wave(requests, ring):
    """Contexts of 512 keys, eight key heads a request: up to 36 requests one wave of the usual kernel holds the
    step's blocks; from 38 to 54 only the kernel with three blocks an SM does; from 56 on neither."""
    keys, got = cut_keys_and_ring(512, requests * 8, held, held_light)
    assert got == ring and keys % 64 == 0
    if ring == 3:
        assert keys == cut_keys(512, requests * 8, held)


def test_without_a_light_kernel_nothing_changes():
    for units in (8, 64, 320, 384, 1000):
        assert cut_keys_and_ring(4096, units, held, lambda cluster: 0) == (cut_keys(4096, units, held), 3)
        assert cut_keys_and_ring(4096, units, held) == (cut_keys(4096, units, held), 3)
    assert LIGHT_COST > 1
