#ifndef SXB_LAMMPS_SHIM_COMM_H
#define SXB_LAMMPS_SHIM_COMM_H
namespace LAMMPS_NS {
class Pair;
class Comm { public: int me, nprocs; void forward_comm(Pair *); void reverse_comm(Pair *); };
}
#endif
