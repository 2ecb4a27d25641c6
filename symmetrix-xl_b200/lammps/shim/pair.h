#ifndef SXB_LAMMPS_SHIM_PAIR_H
#define SXB_LAMMPS_SHIM_PAIR_H
#include "pointers.h"
namespace LAMMPS_NS {
class Pair : protected Pointers {
 public:
  explicit Pair(LAMMPS *lmp) : Pointers(lmp) {}
  virtual void compute(int, int) = 0;
  virtual void settings(int, char **) = 0;
  virtual void coeff(int, char **) = 0;
  virtual double init_one(int, int) { return 0.0; }
  virtual void init_style() {}
  virtual int pack_forward_comm(int, int *, double *, int, int *) { return 0; }
  virtual void unpack_forward_comm(int, int, double *) {}
  virtual int pack_reverse_comm(int, int, double *) { return 0; }
  virtual void unpack_reverse_comm(int, int *, double *) {}
  virtual void *extract(const char *, int &) { return nullptr; }
  double eng_vdwl = 0.0, virial[6] = {0, 0, 0, 0, 0, 0};
  double *eatom = nullptr;
  int comm_forward = 0, comm_reverse = 0;
  int single_enable = 1, restartinfo = 1, one_coeff = 0, manybody_flag = 0, no_virial_fdotr_compute = 0;
 protected:
  void ev_init(int eflag, int vflag) { eflag_global = eflag & 1; eflag_atom = eflag & 2; vflag_global = vflag & 3; vflag_atom = vflag & 4; }
  int allocated = 0, eflag_global = 0, eflag_atom = 0, vflag_global = 0, vflag_atom = 0;
  int **setflag = nullptr;
  double **cutsq = nullptr;
  NeighList *list = nullptr;
};
}    // namespace LAMMPS_NS
#endif
