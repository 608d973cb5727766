"""The few ``mpi4py.MPI`` names the reference touches without sending a message."""
import os


class _NoMPI(RuntimeError):
    def __init__(self, what: str):
        super().__init__(f"{what}: there is no MPI implementation on this machine (mpi4py stand-in)")


class Comm:
    """Type used in ``isinstance(group, MPI.Comm)``; nothing constructs a working one."""

    def Get_rank(self) -> int:
        return int(os.environ.get("RANK", os.environ.get("SLURM_PROCID", "0")))

    def Get_size(self) -> int:
        return int(os.environ.get("WORLD_SIZE", os.environ.get("SLURM_NTASKS", "1")))

    def Barrier(self) -> None:
        # the reference only calls this around its extension build (rank 0 first); with the
        # process group up a torch barrier gives the same ordering
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            dist.barrier()

    def Split(self, color=0, key=0):
        raise _NoMPI("MPI.Comm.Split")

    def __getattr__(self, name):
        raise _NoMPI(f"MPI.Comm.{name}")


class Intracomm(Comm):
    pass


class Request:
    def Wait(self, status=None):
        raise _NoMPI("MPI.Request.Wait")


class Status:
    pass


class memory:  # noqa: N801  (mpi4py spells it in lower case)
    @staticmethod
    def fromaddress(address, nbytes, readonly=False):
        raise _NoMPI("MPI.memory.fromaddress")


FLOAT = "MPI_FLOAT"
BYTE = "MPI_BYTE"
SUM = "MPI_SUM"
IN_PLACE = "MPI_IN_PLACE"
COMM_WORLD = Intracomm()
