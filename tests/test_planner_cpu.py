"""Host planner (tile width, K split, CTA pairs, cluster split-K) exercised without a GPU through
fastnn_b200_plan_query: with no initialised device it plans for a B200's SM and cluster counts."""
import pytest

NN, NT, TN = 0, 1, 2


@pytest.fixture(scope="module")
def plan(built_library):
    import fastnn_b200 as f
    return f.plan_query


def test_large_square_gemms_take_cta_pairs_with_the_widest_tile(plan):
    for layout in (NN, NT, TN):
        p = plan(layout, 8192, 8192, 8192)
        assert p == {"block_n": 512, "split_k": 1, "cta_pair": True, "cluster_k": False}
    for shape in ((NN, 32768, 16384, 4096), (NT, 32768, 4096, 16384), (TN, 4096, 16384, 32768)):
        p = plan(*shape)
        assert p["cta_pair"] and p["block_n"] == 512 and p["split_k"] == 1
    # the 256 x 512 tile only where its waves take less time than those of 256 x 256 tiles
    assert plan(NN, 5120, 4096, 4096)["block_n"] == 256
    assert plan(NN, 4096, 8192, 8192) == {"block_n": 256, "split_k": 1, "cta_pair": True, "cluster_k": False}
    # the row shards of the 8192-row problem over 8 and 4 GPUs: one and two waves of wide tiles
    for rows in (1024, 2048):
        assert plan(NN, rows, 8192, 8192) == {"block_n": 512, "split_k": 1, "cta_pair": True, "cluster_k": False}


def test_transformer_block_forward_shapes_are_not_split(plan):
    for k, n in ((256, 768), (256, 256), (256, 1024), (1024, 256)):
        fwd, dx = plan(NN, 8192, n, k), plan(NT, 8192, k, n)
        for p in (fwd, dx):
            assert p["split_k"] == 1 and not p["cta_pair"] and not p["cluster_k"]
            assert p["block_n"] % 32 == 0 and 32 <= p["block_n"] <= 256


def test_weight_gradients_with_long_k_split_through_the_workspace(plan):
    """dW = X^T . dY with k = 8192 rows and 4-16 output tiles: cut deeper than a cluster can be."""
    for m, n in ((256, 768), (256, 256), (256, 1024), (1024, 256)):
        p = plan(TN, m, n, 8192)
        assert p["split_k"] >= 12 and not p["cluster_k"] and not p["cta_pair"]
        tiles = -(-m // 128) * -(-n // p["block_n"])
        assert 96 <= tiles * p["split_k"] <= 148, "about one wave of CTAs"


def test_mnist_layer_is_cut_inside_clusters(plan):
    p = plan(NN, 512, 256, 784)
    assert p["cluster_k"] and p["split_k"] in (2, 4, 8) and not p["cta_pair"]
    assert (784 + 31) // 32 >= 2 * p["split_k"]


def test_batched_attention_shapes(plan):
    s, o = plan(NT, 128, 128, 32, 512), plan(NN, 128, 32, 128, 512)
    assert s == {"block_n": 128, "split_k": 1, "cta_pair": False, "cluster_k": False}
    assert o == {"block_n": 32, "split_k": 1, "cta_pair": False, "cluster_k": False}


@pytest.mark.parametrize("layout", [NN, NT, TN])
def test_every_plan_is_launchable(plan, layout):
    """Sweep: tile widths are multiples of 32 up to 256 (64 for pairs; 512 only for pairs, only with
    the whole K range per tile and a deep K), every K slice has at least one 32-deep k-block,
    clusters stay within the sizes the kernel reduces over."""
    for m in (1, 100, 128, 500, 4096):
        for n in (1, 32, 100, 260, 4096):
            for k in (1, 31, 64, 1000, 20000):
                for batch in (1, 7):
                    p = plan(layout, m, n, k, batch)
                    assert 32 <= p["block_n"] <= 512 and p["block_n"] % 32 == 0
                    if p["block_n"] > 256:
                        assert p["block_n"] == 512 and p["cta_pair"] and p["split_k"] == 1 and k >= 4096
                    if p["cta_pair"]:
                        assert p["block_n"] % 64 == 0 and m > 128
                    assert 1 <= p["split_k"] <= max(1, -(-k // 32))
                    if p["cluster_k"]:
                        assert p["split_k"] in (2, 4, 8, 16) and not p["cta_pair"]


def test_bad_arguments_are_rejected(plan):
    with pytest.raises(ValueError):
        plan(3, 8, 8, 8)
    with pytest.raises(ValueError):
        plan(NN, 0, 8, 8)
