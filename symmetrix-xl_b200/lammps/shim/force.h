#ifndef SXB_LAMMPS_SHIM_FORCE_H
#define SXB_LAMMPS_SHIM_FORCE_H
namespace LAMMPS_NS { class Force { public: int newton_pair; }; }
#endif
