"""Job configuration schema (text-format ``PS.AppConfig``) and process flags.

Message and field names, types, labels and defaults mirror the reference's schema:
src/proto/app.proto, config.proto, linear_method.proto, neural_network.proto, range.proto,
example.proto, matrix.proto, evaluation.proto, node.proto, task.proto.  A ``.conf`` written for the
reference parses unchanged with :func:`load_app_config`.

Flags follow the gflags surface of the reference (single- or double-dash, ``-flag=value``,
``-flag value``, ``-noflag``): src/system/postoffice.cc:10-24, src/system/van.cc:9-16,
src/system/remote_node.cc:9, src/system/app.cc:6, src/system/ocean.cc:14-17,
src/linear_method/feature_station.cc:14-20, src/linear_method/linear_method.cc:14,
src/data/slot_reader.cc:8, src/data/example_parser.cc:9-14, src/util/filelinereader.cc:13,
src/ps.cc:3.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

from .utils.pbtext import Enum, Field, Message, Schema, dumps, parse, parse_file

F = Field

# ---------------------------------------------------------------- range / node
PbRange = Schema("PbRange", F("begin", "uint64", "required"), F("end", "uint64", "required"))

NodeRole = Enum("Node.Role", SERVER=0, WORKER=1, MANAGER=2, SCHEDULER=3, GROUP=4, UNUSED=5)
Node = Schema("Node", F("role", NodeRole, "required"), F("id", "string"), F("hostname", "string"),
              F("port", "int32"), F("key", PbRange))

# ---------------------------------------------------------------- config.proto
DataFormat = Enum("DataConfig.DataFormat", BIN=1, PROTO=2, TEXT=3)
TextFormat = Enum("DataConfig.TextFormat", PS_DENSE=1, PS_SPARSE=2, PS_SPARSE_BINARY=3, ADFEA=4, LIBSVM=5, TERAFEA=6)
HDFSConfig = Schema("HDFSConfig", F("home", "string"), F("ugi", "string"), F("namenode", "string"))
DataConfig = Schema("DataConfig", F("format", DataFormat, "required"), F("text", TextFormat),
                    F("file", "string", "repeated"), F("hdfs", HDFSConfig), F("range", PbRange),
                    F("ignore_feature_group", "bool"))
ParamInitType = Enum("ParameterInitConfig.Type", ZERO=1, CONSTANT=2, GAUSSIAN=3, FILE=4, CLONE=5)
ParameterInitConfig = Schema("ParameterInitConfig", F("type", ParamInitType, default="ZERO"),
                             F("constant", "double", default=1.0), F("mean", "double", default=0.0),
                             F("std", "double", default=1.0), F("file_name", "string"))
LearningRateType = Enum("LearningRateConfig.Type", CONSTANT=1)
LearningRateConfig = Schema("LearningRateConfig", F("type", LearningRateType), F("eta", "double", default=1.0),
                            F("alpha", "double", default=1.0), F("beta", "double", default=1.0))
PenaltyType = Enum("PenaltyConfig.Type", L1=1, L2=2)
PenaltyConfig = Schema("PenaltyConfig", F("type", PenaltyType, "required"), F("lambda", "double", "repeated"))

# ---------------------------------------------------------------- example / matrix / evaluation
SlotFormat = Enum("SlotInfo.Format", DENSE=1, SPARSE=2, SPARSE_BINARY=3)
SlotInfo = Schema("SlotInfo", F("format", SlotFormat), F("id", "int32"),
                  F("min_key", "uint64", default=0xFFFFFFFFFFFFFFFF), F("max_key", "uint64"),
                  F("nnz_ele", "uint64"), F("nnz_ex", "uint64"))
ExampleInfo = Schema("ExampleInfo", F("slot", SlotInfo, "repeated"), F("num_ex", "uint64"))
MatrixType = Enum("MatrixInfo.Type", DENSE=1, SPARSE=2, SPARSE_BINARY=3)
MatrixInfo = Schema("MatrixInfo", F("type", MatrixType, "required"), F("row_major", "bool", "required"),
                    F("id", "int32"), F("row", PbRange, "required"), F("col", PbRange, "required"),
                    F("nnz", "uint64"), F("sizeof_index", "uint32"), F("sizeof_value", "uint32", "required"))
AUCData = Schema("AUCData", F("tp_key", "int64", "repeated"), F("tp_count", "uint64", "repeated"),
                 F("fp_key", "int64", "repeated"), F("fp_count", "uint64", "repeated"))

# ---------------------------------------------------------------- linear_method.proto
LMSolverConfig = Schema(
    "LM.SolverConfig", F("minibatch_size", "int64", default=0), F("feature_block_ratio", "float", default=0.0),
    F("random_feature_block_order", "bool", default=True), F("prior_fea_group", "int32", "repeated"),
    F("num_iter_for_prior_fea_group", "int32", default=5), F("max_block_delay", "int32", default=0),
    F("max_pass_of_data", "int32", default=10), F("epsilon", "double", default=1e-4),
    F("auc_goodness", "int64", default=100000), F("tail_feature_freq", "int32", default=4),
    F("tail_feature_filter_k", "int32", default=2), F("countmin_k", "int32", default=2),
    F("countmin_n_ratio", "double", default=2.0), F("countmin_n", "double", default=1e8),
    F("max_num_parallel_groups_in_preprocessing", "int32", default=1000),
    F("max_data_buf_size_in_mb", "int32", default=1000), F("eval_interval", "double", default=5))
DarlingConfig = Schema("LM.DarlingConfig", F("delta_init_value", "double", default=1.0),
                       F("delta_max_value", "double", default=5.0),
                       F("kkt_filter_threshold_ratio", "double", default=10.0))
FTRLConfig = Schema("LM.FTRLConfig")
LossType = Enum("LossConfig.Type", SQUARE=1, LOGIT=2, HINGE=3, SQUARE_HINGE=4)
LossConfig = Schema("LM.LossConfig", F("type", LossType, "required"))
LearnerType = Enum("LearnerConfig.Type", GRADIENT_DESCENT=1, PROXIMAL_GRADIENT=2, LBFGS=3)
LearnerConfig = Schema("LM.LearnerConfig", F("type", LearnerType, "required"))
LMConfig = Schema(
    "LM.Config", F("training_data", DataConfig), F("validation_data", DataConfig), F("local_cache", DataConfig),
    F("init_w", ParameterInitConfig), F("model_output", DataConfig), F("model_input", DataConfig),
    F("loss", LossConfig), F("penalty", PenaltyConfig), F("learning_rate", LearningRateConfig),
    F("learner", LearnerConfig), F("solver", LMSolverConfig), F("darling", DarlingConfig), F("ftrl", FTRLConfig))
Progress = Schema("LM.Progress", F("objv", "double"), F("relative_objv", "double"), F("nnz_w", "uint64"),
                  F("violation", "double"), F("nnz_active_set", "uint64"), F("training_auc", "double"),
                  F("training_auc_data", AUCData), F("num_ex_trained", "uint64"), F("acc", "double"),
                  F("total_time", "double"), F("busy_time", "double", "repeated"),
                  F("kkt_threshold", "double"))      # addition of this framework: GPU ranks report the threshold they used
LMCommand = Enum("LM.Call.Command", LOAD_DATA=1, PREPROCESS_DATA=2, UPDATE_MODEL=3, EVALUATE_PROGRESS=4, SAVE_MODEL=5,
                 RECOVER=6, COMPUTE_VALIDATION_AUC=7, REPORT_PROGRESS=8)
LMCall = Schema("LM.Call", F("cmd", LMCommand, "required"), F("key", PbRange), F("kkt_filter_threshold", "double"),
                F("kkt_filter_reset", "bool"), F("fea_grp", "int32", "repeated"), F("hit_cache", "bool"),
                F("progress", Progress),   # REPORT_PROGRESS carries the worker's increment
                # additions of this framework: a task of a scheduled GPU job covers a whole pass
                F("block_order", "int32", "repeated"), F("num_prior", "int32", default=0))

# ---------------------------------------------------------------- neural_network.proto
LayerType = Enum("LayerConfig.Type", NONE=0, FULLY_CONNECTED=1, DATA=2, LOGISTIC_LOSS=3, AUC=4, SPARSE_FULLY_CONNECTED=5)
ActivationType = Enum("ActivationConfig.Type", IDENTITY=0, SIGMOID=1, LOGISTIC=2, SOFTMAX=3, RELU=4, SCALED_TANH=5)
ActivationConfig = Schema("ActivationConfig", F("type", ActivationType, "required"))
LayerConfig = Schema("LayerConfig", F("type", LayerType, "required"), F("name", "string", "required"),
                     F("in", "string", "repeated"), F("out", "string", "repeated"), F("size", "uint32"),
                     F("activation", ActivationConfig), F("minibatch_size", "int32", default=0),
                     F("lr_scale", "double", default=1.0), F("data", DataConfig), F("init", ParameterInitConfig))
NetConfig = Schema("NetConfig", F("name", "string"), F("layer", LayerConfig, "repeated"))
NNSolverType = Enum("NN.SolverConfig.Type", SGD=1)
NNUpdate = Enum("NN.SolverConfig.Update", NORMAL=1, ADAGRAD=2)
NNSolverConfig = Schema("NN.SolverConfig", F("type", NNSolverType, "required"), F("update", NNUpdate),
                        F("lr", LearningRateConfig), F("max_iteration", "int32", default=1000),
                        F("display", "int32", default=100), F("validation", "int32", default=100))
NNConfig = Schema("NN.Config", F("train", NetConfig), F("test", NetConfig), F("solver", NNSolverConfig))

# ---------------------------------------------------------------- app.proto
AppConfig = Schema("AppConfig", F("app_name", "string"), F("parameter_name", "string", "repeated"),
                   F("linear_method", LMConfig), F("neural_network", NNConfig))

# ---------------------------------------------------------------- task.proto
PartitionInfo = Schema("PartitionInfo", F("fea_grp", "int32"), F("key", PbRange))
TaskType = Enum("Task.Type", TERMINATE=1, TERMINATE_CONFIRM=2, REPLY=3, MANAGE=4, CALL_CUSTOMER=5, HEARTBEATING=6)
ManageNodeCmd = Enum("ManageNode.Command", INIT=1, REPLACE=2, REMOVE=3, ADD=4)
ManageNode = Schema("ManageNode", F("cmd", ManageNodeCmd, "required"), F("node", Node, "repeated"))
ManageAppCmd = Enum("ManageApp.Command", ADD=1, REMOVE=2)
ManageApp = Schema("ManageApp", F("cmd", ManageAppCmd, "required"), F("app_config", AppConfig, "required"))
Timestamp = Schema("Timestamp", F("sender", "string", "required"), F("time", "int32", "required"))
SharedParaCmd = Enum("CallSharedPara.Command", PUSH=1, PULL=2)
CallSharedPara = Schema("CallSharedPara", F("cmd", SharedParaCmd, "required"), F("insert_key_freq", "bool"),
                        F("query_key_freq", "int32"), F("insert_key", "bool"), F("countmin_n", "int32"),
                        F("countmin_k", "int32"), F("replica", "bool"), F("backup", Timestamp, "repeated"))
HeartbeatReport = Schema(
    "HeartbeatReport", F("task_id", "int32", default=0), F("hostname", "string"), F("seconds_since_epoch", "uint32"),
    F("total_time_milli", "uint32"), F("busy_time_milli", "uint32"), F("net_in_mb", "uint32"),
    F("net_out_mb", "uint32"), F("process_cpu_usage", "uint32"), F("host_cpu_usage", "uint32"),
    F("process_rss_mb", "uint32"), F("process_virt_mb", "uint32"), F("host_in_use_gb", "uint32"),
    F("host_in_use_percentage", "uint32"), F("host_net_in_bw", "uint32"), F("host_net_out_bw", "uint32"))
Task = Schema("Task", F("type", TaskType, "required"), F("request", "bool", "required", default=False),
              F("customer", "string", "required"), F("time", "int32"), F("wait_time", "int32", default=-1),
              F("has_key", "bool", default=False), F("key_range", PbRange), F("key_signature", "uint32"),
              F("key_channel", "int32"), F("erase_key_cache", "bool", default=False),
              F("uncompressed_size", "uint64", "repeated"), F("msg", "bytes"), F("mng_node", ManageNode),
              F("mng_app", ManageApp), F("shared_para", CallSharedPara), F("linear_method", LMCall),
              F("partition_info", PartitionInfo, "repeated"))


def load_app_config(path: str) -> Message:
    return parse_file(path, AppConfig)


def parse_app_config(text: str) -> Message:
    return parse(text, AppConfig)


def data_files(dc, H) -> list:
    """File patterns of a DataConfig as the host runtime reads them.  With an ``hdfs { home ugi namenode }`` block
    every pattern becomes ``hdfs:<pattern>`` (listed with ``hadoop fs -ls``, read through ``hadoop fs -cat``;
    src/util/file.cc:50-66, 250-300) and this process's hadoop command is set from the block: ``<home>/bin/hadoop``
    (``$HADOOP_HOME`` or the PATH when home is empty), the user of ``ugi`` as ``HADOOP_USER_NAME``, the name node as
    ``-D fs.defaultFS``."""
    import os
    import shlex

    files = list(dc.file)
    if not dc.has("hdfs"):
        return files
    h = dc.hdfs
    home = h.home if h.has("home") and h.home else os.environ.get("HADOOP_HOME", "")
    cmd = shlex.quote(os.path.join(home, "bin", "hadoop")) if home else "hadoop"
    cmd += " fs"
    if h.has("namenode") and h.namenode:
        cmd += " -D " + shlex.quote("fs.defaultFS=" + h.namenode)
    if h.has("ugi") and h.ugi:
        cmd = "HADOOP_USER_NAME=" + shlex.quote(h.ugi.split(",")[0]) + " " + cmd
    H.set_hadoop_fs(cmd)
    return [f if f.startswith("hdfs:") else "hdfs:" + f for f in files]


def parse_node(text: str) -> Message:
    """``role:SCHEDULER,hostname:'127.0.0.1',port:8000,id:'H'`` → Node (src/system/van.h:32-36)."""
    return parse(text, Node)


# ---------------------------------------------------------------- flags
FLAG_DEFAULTS: Dict[str, object] = {
    "num_servers": 0, "num_workers": 0, "num_unused": 0, "num_replicas": 0, "num_threads": 2,
    "app": "../config/rcv1_l1lr.config", "node_file": "./nodes", "report_interval": 0, "verbose": False,
    "log_to_file": False, "parallel_match": False, "enable_fault_tolerance": False,
    "my_node": "", "scheduler": "role:SCHEDULER,hostname:'127.0.0.1',port:8000,id:'H'", "server_master": "",
    "num_retries": 3, "compress_message": True, "print_van": False, "my_rank": -1, "interface": "",
    "key_cache": True, "test_fault_tol": False, "prefetch_job_limit": 64, "less_memory": False,
    "prefetch_mem_limit_kb": 1048576, "mmap_training_data": False, "prefetch_detail": False, "load_limit": 0,
    "load_data_max_mb_per_thread": 2048, "shuffle_fea_id": False, "add_beta_feature": False, "line_limit": 0,
    "log_instant": False,
    # additions of this framework
    "impl": "fused", "gpus": 0, "seed": 0, "timeout_s": 2.0, "checkpoint_dir": "", "checkpoint_interval": 0,
    "trace_file": "", "metrics_file": "", "gpu_scheduler": False,
}


class Flags:
    """gflags-style command line: ``-name value``, ``--name=value``, ``-bool``, ``-nobool``."""

    def __init__(self, **overrides):
        self.__dict__.update(FLAG_DEFAULTS)
        self.__dict__.update(overrides)

    @staticmethod
    def parse(argv: List[str]) -> Tuple["Flags", List[str]]:
        fl, rest, i = Flags(), [], 0
        while i < len(argv):
            a = argv[i]
            if not a.startswith("-") or a in ("-", "--"):
                rest.append(a); i += 1; continue
            name = a.lstrip("-")
            val = None
            if "=" in name:
                name, val = name.split("=", 1)
            if name not in FLAG_DEFAULTS:
                if name.startswith("no") and name[2:] in FLAG_DEFAULTS and isinstance(FLAG_DEFAULTS[name[2:]], bool):
                    setattr(fl, name[2:], False); i += 1; continue
                raise ValueError(f"unknown command line flag '{name}'")
            default = FLAG_DEFAULTS[name]
            if isinstance(default, bool):
                if val is None:
                    val = True
                else:
                    val = val.lower() in ("1", "true", "t", "yes", "y")
            else:
                if val is None:
                    i += 1
                    if i >= len(argv):
                        raise ValueError(f"flag '{name}' needs a value")
                    val = argv[i]
                val = type(default)(val) if not isinstance(default, str) else val
            setattr(fl, name, val)
            i += 1
        return fl, rest

    def as_dict(self) -> Dict[str, object]:
        return {k: getattr(self, k) for k in FLAG_DEFAULTS}


__all__ = [n for n in dir() if not n.startswith("_")]
