"""Trainer callbacks: logging, checkpointing, evaluation, monitoring, schedules and experiment trackers."""

from importlib import import_module

# module -> public names
_EXPORTS = {
    "callback": ("Callback", "CallbackConfig"),
    "checkpointer": ("CheckpointerCallback", "CheckpointRemovalStrategy"),
    "list_checkpointer": ("ListCheckpointerCallback",),
    "console_logger": ("ConsoleLoggerCallback",),
    "config_saver": ("ConfigSaverCallback",),
    "metric_saver": ("MetricSaverCallback",),
    "speed_monitor": ("SpeedMonitorCallback",),
    "garbage_collector": ("GarbageCollectorCallback",),
    "gpu_memory_monitor": ("GPUMemoryMonitorCallback",),
    "gap_monitor": ("GAPMonitorCallback",),
    "stability_monitor": ("StabilityMonitorCallback",),
    "profiler": ("ProfilerCallback",),
    "monkey_patcher": ("MonkeyPatcherCallback",),
    "evaluator_callback": ("EvaluatorCallback", "LMEvaluatorCallbackConfig", "DownstreamEvaluatorCallbackConfig"),
    "batch_size_scheduler": ("BatchSizeSchedulerCallback",),
    "sequence_length_scheduler": ("SequenceLengthSchedulerCallback",),
    "model_merger": ("ModelMergeCallback",),
    "hf_converter": ("HFConverterCallback",),
    "wandb": ("WandBCallback",),
    "comet": ("CometCallback", "CometNotificationSetting"),
    "slack_notifier": ("SlackNotifierCallback", "SlackNotificationSetting"),
    "beaker": ("BeakerCallback",),
}

__all__ = []
for _module, _names in _EXPORTS.items():
    _m = import_module(f"{__name__}.{_module}")
    for _n in _names:
        globals()[_n] = getattr(_m, _n)
        __all__.append(_n)
del _m, _module, _names, _n
