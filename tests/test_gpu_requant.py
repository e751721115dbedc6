"""GPU parity: the FP4 -> affine re-quantiser against its oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from oracle import affine, configs, fp4, requant  # noqa: E402
from tests.helpers import bf16_tensor, max_rel  # noqa: E402


@pytest.mark.parametrize("n,k,group,store", [(96, 512, 128, "float16"), (64, 2880, 64, "float16"), (48, 256, 64, "bfloat16")])
def test_requant_matches_oracle(n, k, group, store):
    """Groups are fitted independently; a group whose candidates tie to the last bit of a squared-error sum may keep a
    different one, so: nearly all groups bit-identical (levels, scale, bias), and the reconstruction error of the
    whole matrix equal to the oracle's to 1e-3."""
    import cachalot_b200 as cb
    rng = np.random.default_rng(n + k)
    p, s = configs.fp4_matrix(rng, n, k)
    w = fp4.dequantize_fp4_weight(p, s)
    o_words, o_s, o_b, o_q = requant.quantize_affine(w, group, 2, store)
    dt = torch.float16 if store == "float16" else torch.bfloat16
    words, gs, gb = cb.requantize_fp4_to_affine(torch.from_numpy(p).cuda(), torch.from_numpy(s).cuda(), bits=2, group_size=group, scale_dtype=dt)
    g_q = affine.unpack_bits(words.cpu().numpy().view(np.uint32), 2, k)
    gs, gb = gs.float().cpu().numpy(), gb.float().cpu().numpy()
    same = (gs == o_s) & (gb == o_b) & np.all(g_q.reshape(-1, group) == o_q.reshape(-1, group), axis=1)
    print(f"requant {n}x{k} g{group} {store}: {same.mean():.4f} of the groups bit-identical")
    assert same.mean() >= 0.97

    def rec(q, sc, bi):
        return (np.repeat(sc, group) * q.reshape(-1) + np.repeat(bi, group)).reshape(n, k)

    e_gpu, e_ref = np.linalg.norm(rec(g_q, gs, gb) - w), np.linalg.norm(rec(o_q, o_s, o_b) - w)
    assert abs(e_gpu - e_ref) <= 1e-3 * e_ref
    # the result is a valid affine matrix for the dequantiser
    deq = cb.dequantize_affine(words, torch.from_numpy(gs).to(dt).cuda(), torch.from_numpy(gb).to(dt).cuda(), bits=2, group_size=group)
    assert np.array_equal(deq.cpu().numpy(), rec(g_q, gs, gb).astype(np.float32))


def test_requantized_bank_runs_and_tracks_the_fp4_bank():
    """An FP4 bank re-quantised to 2 bits on the GPU: same slots and slot table, and the 2-bit layer stays within the
    error the 2-bit fit itself has (relative weight error ~0.39 on uniform codes) of the FP4 layer."""
    import cachalot_b200 as cb
    hidden, inter, n_exp, k = 512, 384, 6, 3
    bank = cb.SlabBank(cb.FP4_FORMAT, hidden, inter, n_exp, layers=1, n_experts=n_exp)
    bank.fill_random(torch.Generator(device="cuda").manual_seed(3))
    two = cb.requantize_bank(bank)
    assert two.fmt.kind == "affine" and two.n_slots == bank.n_slots and torch.equal(two.slot_table, bank.slot_table)
    x = torch.randn((1, hidden), device="cuda").to(torch.bfloat16)
    slots = torch.tensor([[4, 0, 2]], dtype=torch.int32, device="cuda")
    w = torch.tensor([[0.5, 0.3, 0.2]], device="cuda")
    a = cb.moe_forward(x, slots, w, bank, numerics="f32")
    b = cb.moe_forward(x, slots, w, two, numerics="f32")
    assert bool(torch.isfinite(b).all()) and float((a - b).norm() / a.norm()) < 1.0
