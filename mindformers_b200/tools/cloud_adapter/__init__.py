from .cloud_adapter import Local2ObsMonitor, cloud_monitor, mox_adapter
