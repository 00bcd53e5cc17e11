import glob
import os

import pytest

from parameter_server_b200 import config as cfg
from parameter_server_b200.utils import pbtext

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_parse_shipped_configs():
    c = cfg.load_app_config(os.path.join(ROOT, "config", "rcv1_l1lr.conf"))
    lm = c.linear_method
    assert c.app_name == "rcv1" and c.parameter_name == ["rcv1_w"]
    assert lm.training_data.format == "TEXT" and lm.training_data.text == "LIBSVM"
    assert lm.penalty.type == "L1" and lm.penalty.get("lambda") == [1.0]
    assert lm.solver.feature_block_ratio == 4 and lm.solver.max_pass_of_data == 20
    assert lm.solver.minibatch_size == 0              # default ⇒ batch solver
    assert lm.has("darling") and not lm.has("ftrl")
    assert lm.darling.delta_init_value == 5 and lm.darling.kkt_filter_threshold_ratio == 100
    f = cfg.load_app_config(os.path.join(ROOT, "config", "ctr_ftrl.conf")).linear_method
    assert f.has("ftrl") and f.solver.minibatch_size == 100000 and f.learning_rate.alpha == 0.1
    assert f.penalty.get("lambda") == [1.0, 0.1] and f.training_data.ignore_feature_group is True
    d = cfg.load_app_config(os.path.join(ROOT, "config", "ctr_l1lr.conf")).linear_method
    assert d.solver.prior_fea_group == [127, 120] and d.solver.max_block_delay == 8


# the reference checkout, when present, sits beside this repository (or where PSB_REFERENCE_DIR points)
REFERENCE = os.environ.get("PSB_REFERENCE_DIR", os.path.join(os.path.dirname(ROOT), "reference"))


def test_evaluation_and_warm_start_job_files():
    ev = cfg.load_app_config(os.path.join(ROOT, "config", "rcv1_eval.conf")).linear_method
    assert not ev.has("solver") and ev.has("validation_data") and ev.has("model_input")        # selects the evaluation app
    warm = cfg.load_app_config(os.path.join(ROOT, "config", "rcv1_l1lr_warm.conf")).linear_method
    assert warm.init_w.type == "FILE" and warm.init_w.file_name == "output/rcv1" and warm.has("validation_data")


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(REFERENCE, "config", "*.conf"))))
def test_reference_job_files_parse_unchanged(path):
    if path.endswith("mpi.conf"):
        pytest.skip("sourced bash file, not an AppConfig")
    c = cfg.load_app_config(path)
    assert c.has("linear_method") and c.linear_method.loss.type == "LOGIT"


def test_defaults_and_presence():
    c = cfg.parse_app_config('linear_method { solver { } }')
    s = c.linear_method.solver
    assert s.random_feature_block_order is True and s.epsilon == 1e-4 and s.tail_feature_freq == 4
    assert s.countmin_n == 1e8 and s.eval_interval == 5 and s.auc_goodness == 100000
    assert c.linear_method.init_w.type == "ZERO" and not c.linear_method.has("init_w")
    assert c.linear_method.darling.delta_max_value == 5.0


def test_grammar_variants_roundtrip():
    text = '''
      app_name: "a" "b"   # adjacent strings concatenate
      parameter_name: 'x'; parameter_name: "y\\n",
      linear_method: { penalty < type: 1 lambda: [1, 2.5e-1] > loss { type: LOGIT }
        training_data { format: TEXT file: ["p1", "p2"] range { begin: 0 end: 0xFFFFFFFFFFFFFFFF } } }
    '''
    c = cfg.parse_app_config(text)
    assert c.app_name == "ab" and c.parameter_name == ["x", "y\n"]
    assert c.linear_method.penalty.type == "L1" and c.linear_method.penalty.get("lambda") == [1.0, 0.25]
    assert c.linear_method.training_data.range.end == 2**64 - 1
    again = cfg.parse_app_config(pbtext.dumps(c))
    assert again == c


@pytest.mark.parametrize("bad", [
    'no_such_field: 1', 'linear_method { loss { type: NOPE } }', 'linear_method { loss { } }',
    'linear_method { solver { max_pass_of_data: 99999999999 } }', 'app_name: unquoted', 'linear_method { ',
])
def test_errors(bad):
    with pytest.raises(ValueError):
        cfg.parse_app_config(bad)


def test_nn_config():
    c = cfg.parse_app_config('''neural_network { train { name: "t" layer { type: DATA name: "d" out: "x" out: "y" minibatch_size: 128 }
       layer { type: FULLY_CONNECTED name: "fc" in: "x" out: "h" size: 64 activation { type: RELU } } }
       solver { type: SGD update: ADAGRAD lr { alpha: 0.1 beta: 1 } max_iteration: 10 } }''')
    layers = c.neural_network.train.layer
    assert [l.type for l in layers] == ["DATA", "FULLY_CONNECTED"] and layers[1].get("in") == ["x"]
    assert c.neural_network.solver.update == "ADAGRAD" and c.neural_network.solver.display == 100


def test_flags():
    fl, rest = cfg.Flags.parse(["-num_servers", "2", "--num_workers=2", "-my_rank", "3", "-verbose", "-nokey_cache",
                                "-app", "x.conf", "-scheduler", "role:SCHEDULER,hostname:'127.0.0.1',port:2060,id:'H'",
                                "extra"])
    assert (fl.num_servers, fl.num_workers, fl.my_rank, fl.verbose, fl.key_cache, fl.app) == (2, 2, 3, True, False, "x.conf")
    assert rest == ["extra"] and fl.compress_message is True and fl.prefetch_mem_limit_kb == 1048576
    n = cfg.parse_node(fl.scheduler)
    assert n.role == "SCHEDULER" and n.port == 2060 and n.id == "H"
    with pytest.raises(ValueError):
        cfg.Flags.parse(["-bogus", "1"])
