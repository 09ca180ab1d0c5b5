from .heartbeat import HeartbeatMonitor, RankFailure
from .elastic import ElasticRunner, run_with_restarts
