/* -*- c++ -*- ----------------------------------------------------------
   pair_style symmetrix/mace/b200: compact two-layer MACE models evaluated on one B200 per MPI rank
   through the C ABI of libsymmetrix_b200 (include/symmetrix_b200.h).

   Counterpart of the reference's pair styles symmetrix/mace and symmetrix/mace/kk in their
   message-passing mode (pair_symmetrix/pair_symmetrix_mace.cpp:443-646,
   pair_symmetrix/pair_symmetrix_mace_kokkos.cpp:1285-1938): the rank's owned atoms are the receivers,
   its ghost atoms are feature-only nodes; the hidden features H1 travel to the ghosts with LAMMPS'
   forward communication, their adjoints come back with the reverse communication, and LAMMPS' own
   reverse communication of f returns the ghost forces.
------------------------------------------------------------------------- */

#ifdef PAIR_CLASS
// clang-format off
PairStyle(symmetrix/mace/b200,PairSymmetrixMACEB200);
// clang-format on
#else

#ifndef LMP_PAIR_SYMMETRIX_MACE_B200_H
#define LMP_PAIR_SYMMETRIX_MACE_B200_H

#include <cstdint>
#include <string>
#include <vector>

#include "pair.h"

struct sxb_evaluator;

namespace LAMMPS_NS {

class PairSymmetrixMACEB200 : public Pair {
 public:
  PairSymmetrixMACEB200(class LAMMPS *);
  ~PairSymmetrixMACEB200() override;

  void compute(int, int) override;
  void settings(int, char **) override;
  void coeff(int, char **) override;
  double init_one(int, int) override;
  void init_style() override;
  int pack_forward_comm(int, int *, double *, int, int *) override;
  void unpack_forward_comm(int, int, double *) override;
  int pack_reverse_comm(int, int, double *) override;
  void unpack_reverse_comm(int, int *, double *) override;
  void *extract(const char *, int &) override;

 protected:
  void allocate();
  void rebuild_graph();
  void check(int status, const char *what);

  sxb_evaluator *evaluator = nullptr;
  std::string prediction_head;
  int device_ordinal = -1;        // -1: MPI rank modulo the number of visible devices
  double r_cut = 0.0;
  int row_floats = 0;             // num_LM * num_channels: one atom's H1 / H1_adj row

  std::vector<int> mace_types;    // LAMMPS type - 1 -> element slot of the model
  uint64_t generation = 0;        // token of the graph the evaluator holds
  int graph_nlocal = 0, graph_nall = 0;

  // host staging of one step
  std::vector<int> node_types, num_neigh, neigh_indices;
  std::vector<double> positions;  // [nall][3]
  std::vector<float> rows;        // [nall][row_floats]: H1 going forward, H1_adj coming back
  std::vector<double> energies, forces;

  // Run-to-date counters read by `compute symmetrix/timing` through extract(), under the names the
  // reference's pair styles publish (pair_symmetrix/pair_symmetrix_mace.cpp:84-105): the whole pair call,
  // and the hidden-state exchange (staging out of and into the device included) forward and reverse.
  // The pair call is timed only while a compute has raised symmetrix_timing_enabled.
  double execution_pair_seconds = 0.0, execution_pair_evaluation_count = 0.0, execution_timing_enabled = 0.0;
  double execution_mpi_hidden_state_forward_seconds = 0.0, execution_mpi_hidden_state_reverse_seconds = 0.0;
  double execution_mpi_hidden_state_seconds = 0.0;
  double execution_mpi_hidden_state_forward_calls = 0.0, execution_mpi_hidden_state_reverse_calls = 0.0;
};

}    // namespace LAMMPS_NS

#endif
#endif
