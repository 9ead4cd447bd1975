"""Configuration and invocation of `musa_graph_optimizer`.

Keeps the function names and semantics of the reference's helpers
(python/_graph_optimizer.py:129-271 of the reference project), which edit
`ConfigProto.graph_options.rewrite_options`: the optimizer is listed under
`custom_optimizers` with a `parameter_map`, optionally also under `optimizers`,
and `disabled_fusion_patterns` is a comma-joined string of pattern names (or
"all").  TensorFlow's ConfigProto is not available in this build, so the same
structure is kept by `RewriteOptions`, and `optimize_graph_def` runs the C++
optimizer on serialised GraphDef bytes (what Grappler would do with the same
parameters).
"""
import ctypes
import json

from . import _loader

MUSA_GRAPH_OPTIMIZER_NAME = "musa_graph_optimizer"
DISABLED_FUSION_PATTERNS_PARAM = "disabled_fusion_patterns"


class CustomOptimizer:
    def __init__(self, name):
        self.name = name
        self.parameter_map = {}


class RewriteOptions:
    """The two fields of tensorflow.RewriterConfig that the helpers touch."""

    def __init__(self):
        self.custom_optimizers = []
        self.optimizers = []
        self.min_graph_nodes = 0


class GraphOptimizerConfig:
    """Stand-in for ConfigProto: `config.graph_options.rewrite_options`."""

    class _GraphOptions:
        def __init__(self):
            self.rewrite_options = RewriteOptions()

    def __init__(self):
        self.graph_options = GraphOptimizerConfig._GraphOptions()


def _get_rewrite_options(config):
    return config.graph_options.rewrite_options


def _find_custom(rewrite_options):
    for opt in rewrite_options.custom_optimizers:
        if opt.name == MUSA_GRAPH_OPTIMIZER_NAME:
            return opt
    return None


def _normalize_fusion_patterns(patterns):
    """A name, a comma-separated string, an iterable of names, or "all" ->
    de-duplicated list of trimmed names (order kept)."""
    if patterns is None:
        return []
    if isinstance(patterns, str):
        items = patterns.split(",")
    else:
        items = []
        for p in patterns:
            items.extend(str(p).split(","))
    out = []
    for item in items:
        name = item.strip()
        if not name:
            continue
        if name.lower() == "all":
            return ["all"]
        if name not in out:
            out.append(name)
    return out


def set_musa_graph_optimizer_enabled(config=None, enabled=True,
                                     add_to_optimizer_list=False,
                                     disabled_fusion_patterns=None):
    """Enable or disable `musa_graph_optimizer` on a config; returns it."""
    if config is None:
        config = GraphOptimizerConfig()
    ro = _get_rewrite_options(config)
    ro.custom_optimizers = [o for o in ro.custom_optimizers
                            if o.name != MUSA_GRAPH_OPTIMIZER_NAME]
    if enabled:
        custom = CustomOptimizer(MUSA_GRAPH_OPTIMIZER_NAME)
        ro.custom_optimizers.append(custom)
        if disabled_fusion_patterns is not None:
            names = _normalize_fusion_patterns(disabled_fusion_patterns)
            if names:
                custom.parameter_map[DISABLED_FUSION_PATTERNS_PARAM] = ",".join(names)
        if add_to_optimizer_list and MUSA_GRAPH_OPTIMIZER_NAME not in ro.optimizers:
            ro.optimizers.append(MUSA_GRAPH_OPTIMIZER_NAME)
    else:
        ro.optimizers = [o for o in ro.optimizers if o != MUSA_GRAPH_OPTIMIZER_NAME]
    return config


def enable_musa_graph_optimizer(config=None, add_to_optimizer_list=False,
                                disabled_fusion_patterns=None):
    return set_musa_graph_optimizer_enabled(config, True, add_to_optimizer_list,
                                            disabled_fusion_patterns)


def disable_musa_graph_optimizer(config=None):
    return set_musa_graph_optimizer_enabled(config, False)


def is_musa_graph_optimizer_enabled(config):
    return _find_custom(_get_rewrite_options(config)) is not None


def set_musa_disabled_fusion_patterns(config=None, patterns=None,
                                      add_to_optimizer_list=False):
    """Set (replace) the disabled patterns; enables the optimizer if needed."""
    if config is None or not is_musa_graph_optimizer_enabled(config):
        config = enable_musa_graph_optimizer(config, add_to_optimizer_list)
    custom = _find_custom(_get_rewrite_options(config))
    names = _normalize_fusion_patterns(patterns)
    if names:
        custom.parameter_map[DISABLED_FUSION_PATTERNS_PARAM] = ",".join(names)
    else:
        custom.parameter_map.pop(DISABLED_FUSION_PATTERNS_PARAM, None)
    return config


def disable_musa_fusion_patterns(patterns, config=None, add_to_optimizer_list=False):
    return set_musa_disabled_fusion_patterns(config, patterns, add_to_optimizer_list)


def clear_musa_disabled_fusion_patterns(config=None, add_to_optimizer_list=False):
    return set_musa_disabled_fusion_patterns(config, None, add_to_optimizer_list)


def get_musa_disabled_fusion_patterns(config):
    custom = _find_custom(_get_rewrite_options(config))
    if custom is None:
        return []
    return _normalize_fusion_patterns(
        custom.parameter_map.get(DISABLED_FUSION_PATTERNS_PARAM, ""))


# ------------------------------------------------------------- invocation --

def _graph_lib():
    lib = _loader.get_library()
    if not getattr(lib, "_graph_bound", False):
        lib.MusaGraphOptimizerName.restype = ctypes.c_char_p
        lib.MusaGraphOptimizerRun.restype = ctypes.c_int
        lib.MusaGraphOptimizerRun.argtypes = [
            ctypes.c_char_p, ctypes.c_size_t, ctypes.c_char_p,
            ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_size_t),
            ctypes.c_char_p, ctypes.c_size_t]
        lib.MusaGraphOptimizerFree.argtypes = [ctypes.c_void_p]
        lib.MusaGraphOptimizerFree.restype = None
        lib.MusaGraphOptimizerListPatterns.restype = ctypes.c_int
        lib.MusaGraphOptimizerListPatterns.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
        lib.MusaGraphSetPatternEnabled.restype = ctypes.c_int
        lib.MusaGraphSetPatternEnabled.argtypes = [ctypes.c_char_p, ctypes.c_int]
        lib.TFMusaSetGraphDumpConfig.restype = None
        lib.TFMusaSetGraphDumpConfig.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.c_int,
                                                 ctypes.c_int]
        lib.TFMusaClearGraphDumpConfig.restype = None
        lib.TFMusaGetGraphDumpDirectory.restype = ctypes.c_char_p
        lib.TFMusaSetAllowGrowth.restype = None
        lib.TFMusaSetAllowGrowth.argtypes = [ctypes.c_int]
        lib._graph_bound = True
    return lib


def list_fusion_patterns():
    """[(name, priority, kernel_available)], highest priority first."""
    buf = ctypes.create_string_buffer(4096)
    _graph_lib().MusaGraphOptimizerListPatterns(buf, len(buf))
    out = []
    for line in buf.value.decode().splitlines():
        name, prio, avail = line.split(":")
        out.append((name, int(prio), avail == "1"))
    return out


def optimize_graph_def(graph_def_bytes, config=None, parameters=None):
    """Run `musa_graph_optimizer` over serialised GraphDef bytes.

    `config`: a GraphOptimizerConfig; when given and the optimizer is not
    enabled on it, the bytes are returned unchanged.  `parameters`: a
    parameter_map dict that overrides the config's.  Returns (bytes, report)."""
    params = {}
    if config is not None:
        custom = _find_custom(_get_rewrite_options(config))
        if custom is None:
            return bytes(graph_def_bytes), {"applied": 0, "skipped": "optimizer not enabled"}
        params.update(custom.parameter_map)
    if parameters:
        params.update(parameters)
    text = ";".join("%s=%s" % kv for kv in params.items()).encode()
    lib = _graph_lib()
    out = ctypes.c_void_p()
    out_n = ctypes.c_size_t()
    report = ctypes.create_string_buffer(4096)
    data = bytes(graph_def_bytes)
    rc = lib.MusaGraphOptimizerRun(data, len(data), text, ctypes.byref(out),
                                   ctypes.byref(out_n), report, len(report))
    if rc != 0:
        from .errors import InternalError, InvalidArgumentError
        cls = InvalidArgumentError if rc == 3 else InternalError
        raise cls("musa_graph_optimizer: %s (code %d)" % (report.value.decode(), rc))
    try:
        result = ctypes.string_at(out, out_n.value)
    finally:
        lib.MusaGraphOptimizerFree(out)
    return result, json.loads(report.value.decode())


# -------------------------------------------------- runtime configuration --
# The reference's python/_graph_optimizer.py:275-345 and python/__init__.py:59.

def set_musa_graph_dump_config(enabled=True, dump_dir=".", dump_text=False, dump_slim=False):
    """Configure GraphDef dumping of `musa_graph_optimizer`; overrides the
    MUSA_DUMP_GRAPHDEF, MUSA_DUMP_GRAPHDEF_DIR, MUSA_DUMP_GRAPHDEF_TEXT and
    MUSA_DUMP_GRAPHDEF_SLIM environment variables for this process."""
    _graph_lib().TFMusaSetGraphDumpConfig(
        int(bool(enabled)), ("." if dump_dir is None else str(dump_dir)).encode(),
        int(bool(dump_text)), int(bool(dump_slim)))


def enable_musa_graph_dump(dump_dir=".", dump_text=False, dump_slim=False):
    set_musa_graph_dump_config(True, dump_dir, dump_text, dump_slim)


def disable_musa_graph_dump():
    set_musa_graph_dump_config(enabled=False)


def clear_musa_graph_dump_config():
    """Drop the override and fall back to the environment variables."""
    _graph_lib().TFMusaClearGraphDumpConfig()


def is_musa_graph_dump_enabled():
    return bool(_graph_lib().TFMusaGraphDumpIsEnabled())


def get_musa_graph_dump_directory():
    return _graph_lib().TFMusaGetGraphDumpDirectory().decode()


def is_musa_graph_dump_text_enabled():
    return bool(_graph_lib().TFMusaGraphDumpTextIsEnabled())


def is_musa_graph_dump_slim_enabled():
    return bool(_graph_lib().TFMusaGraphDumpSlimIsEnabled())


def set_musa_allow_growth(enabled=True):
    """Ask for on-demand growth of the device memory pool instead of one
    up-front reservation (read by the platform registration; the
    TF_FORCE_GPU_ALLOW_GROWTH environment variable wins when it is set)."""
    _graph_lib().TFMusaSetAllowGrowth(int(bool(enabled)))


def get_musa_allow_growth():
    return bool(_graph_lib().TFMusaGetAllowGrowth())
