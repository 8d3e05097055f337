"""A target and a drafter built straight from GGUF files (mapped, never copied through Python) behave exactly like the
same tensors handed over as a table."""
import numpy as np
import pytest

import ggufgen
import modelgen
from dflb import pkg

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("v2", [False, True])
def test_model_and_drafter_from_gguf_equal_table_built_ones(tmp_path, v2):
    arch = modelgen.tiny_arch()
    T = modelgen.target_tensors(arch, seed=3)
    cfg = modelgen.tiny_dflash_config(arch, selector_rank=256 if v2 else 0, selector_top_k=16 if v2 else 0)
    D = modelgen.drafter_tensors(arch, cfg, seed=4)
    tp, dp = tmp_path / "target.gguf", tmp_path / "drafter.gguf"
    ggufgen.write_gguf(tp, "qwen35", ggufgen.arch_meta(arch), T)
    ggufgen.write_gguf(dp, "dflash" if v2 else "dflash-draft", ggufgen.drafter_meta(cfg, v2), ggufgen.v2_names(D) if v2 else D)
    gt, gd = pkg.GGUF(tp), pkg.GGUF(dp)
    m_file = pkg.Model.from_gguf(gt)
    d_file = pkg.Drafter.from_gguf(m_file, gd)
    gt.close(); gd.close()                      # the library keeps its own device copies (and host codebooks)
    m_tab = pkg.Model(arch, T)
    d_tab = pkg.Drafter(m_tab, cfg, D)
    assert m_file.verify_weight_bytes() == m_tab.verify_weight_bytes() and d_file.weight_bytes() == d_tab.weight_bytes()
    prompt = np.random.default_rng(2).integers(0, arch.vocab_size, size=20)
    outs = []
    for m, d in ((m_file, d_file), (m_tab, d_tab)):
        ids = d.layer_ids()
        sess, scr, ds = pkg.Session(m, 64), pkg.Scratch(m, 16, len(ids)), pkg.DSession(d, 64)
        logits, _ = pkg.prefill(m, sess, scr, ids, prompt, 0, feed_drafter=ds)
        toks, dl = ds.draft_block(int(np.argmax(logits)), 20, want_logits=True)
        outs.append((logits, toks, dl))
        for x in (sess, scr, ds):
            x.close()
    assert outs[0][0].tobytes() == outs[1][0].tobytes()
    assert np.array_equal(outs[0][1], outs[1][1]) and outs[0][2].tobytes() == outs[1][2].tobytes()
    for x in (d_file, d_tab, m_file, m_tab):
        x.close()
