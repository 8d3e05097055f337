"""Session snapshots: a session restored from a snapshot continues bitwise like the session it was taken from
(the reference's guarantee for SessionSnapshot, metal_forward/session.rs:57-62), the drafter's context tail follows its
capture-window rule (metal_dflash.rs:103-140), and mismatching snapshots are refused."""
import numpy as np
import pytest

import modelgen
from dflb import pkg

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def world():
    arch = modelgen.tiny_arch()
    T = modelgen.target_tensors(arch, seed=3)
    gm = pkg.Model(arch, T)
    yield arch, gm
    gm.close()


def continue_block(gm, gd, sess, scr, ds, carry, pos, block):
    toks, dl = ds.draft_block(carry, pos, want_logits=True)
    am, gap, logits = pkg.packed_verify(gm, sess, scr, gd.layer_ids(), block, pos, want_logits=True)
    states = [np.concatenate(sess.read_gdn_state(g)) for g in range(2)]
    return toks, dl, am, logits, states


@pytest.mark.parametrize("all_swa", [False, True])
def test_restored_session_continues_bitwise(world, all_swa):
    arch, gm = world
    cfg = modelgen.tiny_dflash_config(arch, swa=[1, 1] if all_swa else [1, 0])
    gd = pkg.Drafter(gm, cfg, modelgen.drafter_tensors(arch, cfg, seed=4))
    ids = gd.layer_ids()
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, arch.vocab_size, size=37)
    block = rng.integers(0, arch.vocab_size, size=16)
    sess, scr, ds = pkg.Session(gm, 128), pkg.Scratch(gm, 16, len(ids)), pkg.DSession(gd, 128)
    logits, _ = pkg.prefill(gm, sess, scr, ids, prompt, 0, feed_drafter=ds)
    carry = int(np.argmax(logits))
    blob = pkg.session_snapshot(gm, sess, ds)
    ident = pkg.snapshot_identity(gm, sess)
    assert ident.layout_version == 2 and ident.kv_storage_kind == 1 and ident.kv_bytes_per_token == 2 * ident.kv_dim_elements
    # the drafter tail: all 37 columns, or the last swa_window (8) of an all-sliding-window drafter
    kv_dim = cfg.n_kv_heads * cfg.head_dim
    cols = 8 if all_swa else 37
    target_part = blob.size - (cols * 4 + cfg.n_layer * 2 * cols * kv_dim * 4)
    no_drafter = pkg.session_snapshot(gm, sess, None)
    assert no_drafter.size == target_part
    want = continue_block(gm, gd, sess, scr, ds, carry, 37, block)
    # restore into fresh sessions of another capacity
    sess2, scr2, ds2 = pkg.Session(gm, 96), pkg.Scratch(gm, 16, len(ids)), pkg.DSession(gd, 64)
    pkg.session_restore_snapshot(gm, sess2, ds2, blob)
    assert sess2.kv_n_pos == 37 and ds2.ctx_len == cols
    got = continue_block(gm, gd, sess2, scr2, ds2, carry, 37, block)
    assert np.array_equal(got[0], want[0]) and got[1].tobytes() == want[1].tobytes()          # drafts and draft logits
    assert np.array_equal(got[2], want[2]) and got[3].tobytes() == want[3].tobytes()          # verify argmax and logits
    assert all(a.tobytes() == b.tobytes() for a, b in zip(got[4], want[4]))                   # recurrent state
    # refusals
    with pytest.raises(pkg.DflError):
        pkg.session_restore_snapshot(gm, pkg.Session(gm, 128, kv_f16=False), None, no_drafter)    # identity: KV storage kind
    with pytest.raises(pkg.DflError) as e:
        pkg.session_restore_snapshot(gm, pkg.Session(gm, 32), None, no_drafter)                   # prefix exceeds capacity
    assert e.value.name == "KV_STATE"
    with pytest.raises(pkg.DflError):
        pkg.session_restore_snapshot(gm, pkg.Session(gm, 128), None, no_drafter[:-8])             # section length
    bad = no_drafter.copy()
    bad[0] ^= 0xFF
    with pytest.raises(pkg.DflError):
        pkg.session_restore_snapshot(gm, pkg.Session(gm, 128), None, bad)                         # magic
    with pytest.raises(pkg.DflError):
        pkg.session_restore_snapshot(gm, pkg.Session(gm, 128), pkg.DSession(gd, 128), no_drafter)  # no drafter context inside
    fresh = pkg.Session(gm, 128)
    before = [np.concatenate(fresh.read_gdn_state(g)).tobytes() for g in range(2)]
    with pytest.raises(pkg.DflError) as e:
        pkg.session_restore_snapshot(gm, fresh, pkg.DSession(gd, 4), blob)                        # drafter tail does not fit
    assert e.value.name == "CTX_OVERFLOW"
    # the refusal came before the first copy: the target session is as it was
    assert fresh.kv_n_pos == 0 and not fresh.poisoned
    assert [np.concatenate(fresh.read_gdn_state(g)).tobytes() for g in range(2)] == before
    # a drafter of another shape (one more layer) does not accept this drafter's section
    cfg3 = modelgen.tiny_dflash_config(arch, n_layer=3, swa=[1, 1, 1] if all_swa else [1, 1, 0])
    gd3 = pkg.Drafter(gm, cfg3, modelgen.drafter_tensors(arch, cfg3, seed=4))
    with pytest.raises(pkg.DflError):
        pkg.session_restore_snapshot(gm, fresh, pkg.DSession(gd3, 128), blob)
    assert fresh.kv_n_pos == 0
    gd3.close()
    gd.close()
