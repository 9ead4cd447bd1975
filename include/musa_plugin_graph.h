/* C ABI of the graph optimizer ("musa_graph_optimizer") inside
 * libmusa_plugin_kernels.so: the fusion-pattern registry and its driver,
 * operating on a serialised TensorFlow GraphDef.
 *
 * In the reference the optimizer is a Grappler CustomGraphOptimizer registered
 * with REGISTER_GRAPH_OPTIMIZER_AS(MusaGraphOptimizer, "musa_graph_optimizer")
 * (musa_ext/mu/optimizer/musa_graph_optimizer.cc:6279) whose Optimize() hands
 * `item.graph` to OptimizeFusion (:5843-5995).  The entry point below is that
 * step with the GraphDef crossing the boundary as protobuf wire bytes, so the
 * Grappler glue reduces to SerializeToString / ParseFromString around one call.
 */
#ifndef MUSA_PLUGIN_GRAPH_H_
#define MUSA_PLUGIN_GRAPH_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* "musa_graph_optimizer": the name a ConfigProto lists under
 * graph_options.rewrite_options.custom_optimizers (python/_graph_optimizer.py:18). */
const char* MusaGraphOptimizerName(void);

/* Runs the enabled fusion patterns to a fixed point over `graph_def`
 * (GraphDef wire bytes) and returns the rewritten GraphDef in a buffer owned by
 * the library (*out_graph_def, *out_size; release with MusaGraphOptimizerFree).
 * `params`: the optimizer's parameter_map as "key=value;key=value", e.g.
 * "disabled_fusion_patterns=MusaAdamMixedFusion, musabiasaddrelufusion" or
 * "disabled_fusion_patterns=all"; NULL for defaults.  `report` (optional)
 * receives a JSON summary: applied / fallbacks / iterations / per-pattern counts.
 * Returns 0, or a tensorflow::error code: 3 INVALID_ARGUMENT (malformed bytes,
 * unknown parameter; the message is in `report`), 13 INTERNAL.
 * Replaces MusaGraphOptimizer::Init + OptimizeFusion
 * (musa_ext/mu/optimizer/musa_graph_optimizer.cc:5414-5478, 5843-5995). */
int MusaGraphOptimizerRun(const void* graph_def, size_t graph_def_size,
                          const char* params, void** out_graph_def,
                          size_t* out_size, char* report, size_t report_cap);
void MusaGraphOptimizerFree(void* graph_def);

/* Registered patterns, highest priority first, as "name:priority:kernel\n"
 * lines; returns their number.  (FusionPatternManager::GetSortedPatterns,
 * musa_ext/graph/fusion/fusion_pattern_manager.h:109-111.) */
int MusaGraphOptimizerListPatterns(char* buf, size_t cap);

/* FusionPatternManager::SetPatternEnabled
 * (musa_ext/graph/fusion/fusion_pattern_manager.h:116-117); 5 NOT_FOUND for an
 * unknown name. */
int MusaGraphSetPatternEnabled(const char* pattern_name, int enabled);

/* GraphDef dumps around the fusion pass: with dumping on, every optimizer run
 * writes <dir>/musa_graph_optimizer_<id:04>_{initial,before_fusion,
 * after_fusion,final}.pb (wire bytes, unknown fields included), plus .slim.pb
 * (scalar attrs only) and .pbtxt (name / op / input / device / scalar attrs)
 * when asked.  The override set here wins over the environment variables
 * MUSA_DUMP_GRAPHDEF, MUSA_DUMP_GRAPHDEF_DIR, MUSA_DUMP_GRAPHDEF_TEXT,
 * MUSA_DUMP_GRAPHDEF_SLIM until it is cleared.  Same names and arguments as
 * the reference (musa_ext/mu/runtime_config_c_api.h:11-17, defined at
 * musa_ext/mu/optimizer/graph_utils.cc:552-589). */
void TFMusaSetGraphDumpConfig(int enabled, const char* dump_dir, int dump_text,
                              int dump_slim);
void TFMusaClearGraphDumpConfig(void);
int TFMusaGraphDumpIsEnabled(void);
const char* TFMusaGetGraphDumpDirectory(void);
int TFMusaGraphDumpTextIsEnabled(void);
int TFMusaGraphDumpSlimIsEnabled(void);

/* Allow-growth switch that the platform registration reads when TensorFlow
 * sets up the device allocator (musa_ext/mu/runtime_config_c_api.h:6, defined at
 * musa_ext/mu/device_register.cc:155-157).  TFMusaGetAllowGrowth returns the
 * effective value: TF_FORCE_GPU_ALLOW_GROWTH=true|false wins over the call
 * (musa_ext/mu/device_register.cc:55-67); the getter has no counterpart symbol
 * in the reference, which reads the value in-process. */
void TFMusaSetAllowGrowth(int enabled);
int TFMusaGetAllowGrowth(void);

#ifdef __cplusplus
}
#endif

#endif /* MUSA_PLUGIN_GRAPH_H_ */
